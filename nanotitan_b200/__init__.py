"""nanotitan_b200: a Blackwell-native (sm_100a) MoE language-model training stack.

Framework layer in PyTorch (config, model, DP/PP/EP, train loop); hot paths are
hand-written CUDA kernels in `nanotitan_b200/csrc`, loaded as the `nanotitan_cuda`
extension through `nanotitan_b200.ops.ext`.
"""
__version__ = "0.1.0"
