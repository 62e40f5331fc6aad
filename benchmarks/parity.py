"""Loss parity against the reference's own code, from one set of weights on the same batches.

`run_parity` builds the reference model (installed under baseline/_ref, fp32 parameters, its torch
MoE backend) and this framework's model (bf16 parameters + fp32 master weights, sm_100a kernels),
copies the reference's `state_dict()` into ours - the key layout is the same
(reference: src/model/model.py:219-269) - and trains both with their own
`PipelineParallel.train_step` (reference: src/parallel/pp.py:30-134) on identical batches.
It returns both cross-entropy curves and their largest gaps.  The reference's fp32 run is the
oracle; ours computes in bf16, so the curves agree to bf16 rounding, not bitwise.

    python bench.py --parity [--config moe] [--parity-steps 20]      # full-size models, 1 GPU
"""
from __future__ import annotations

import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
for extra in (ROOT, ROOT / "baseline"):
    if str(extra) not in sys.path:
        sys.path.insert(0, str(extra))


def run_parity(model_kw: dict, batch: int, steps: int, lr: float, seed: int = 42) -> dict:
    import ref_harness

    why = ref_harness.available()
    if why is not None:
        return {"unavailable": why}
    import torch

    # ---- the reference, in fp32, through its own code
    ref_kw = dict(model_kw, dtype="float32")
    ref_cfg, ref_dims, ref_model, ref_step, ref_opt = ref_harness.build(ref_kw, batch, 1, 1, 1, 1, lr, seed)
    weights = {k: v.detach().clone() for k, v in ref_model.state_dict().items()}

    # ---- ours, started from the same weights
    from nanotitan_b200.config import AppConfig
    from nanotitan_b200.models.cuda_backend import CUDAMoEBackend
    from nanotitan_b200.parallel_dims import get_parallel_dims
    from nanotitan_b200.train import build_training
    from nanotitan_b200.utils.checkpoint import load_full_state

    cfg = AppConfig.model_validate(dict(
        run_name="parity", max_steps=steps, model=dict(model_kw, moe_backend="cuda", dtype="bfloat16"),
        trainer=dict(device_id=0, eval_every_step=-1, per_device_batch_size=batch, seed=seed),
        data=dict(num_workers=1, train_tokens_path="unused", val_tokens_path="unused"),
        optim=dict(type="adam", lr=lr),
        runtime=dict(name="parity", dp_size=1, pp_size=1, ep_size=1, num_microbatches=1, bucket_size=25),
    ))
    dims = get_parallel_dims(cfg.runtime)
    model, _, step, optimizer = build_training(cfg, dims)
    load_full_state(model, weights)
    own = dict(model.named_parameters())
    optimizer.set_master_weights({id(own[k]): v for k, v in weights.items() if k in own})
    # the reference's torch backend lets the load-balancing loss reach the tokens; match it
    before = CUDAMoEBackend.aux_to_tokens
    CUDAMoEBackend.aux_to_tokens = True
    try:
        gen = torch.Generator().manual_seed(seed)
        seq, vocab = cfg.model.max_seq_len, cfg.model.vocab_size
        ref_curve, our_curve, ref_aux, our_aux = [], [], [], []
        for _ in range(steps):
            ids = torch.randint(0, vocab, (batch, seq + 1), generator=gen, dtype=torch.int64)
            x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
            m_ref = ref_step.train_step(ref_model, (x, y), ref_opt)
            m_our = step.train_step(model, (x, y), optimizer)
            ref_curve.append(float(m_ref["train/ce_loss"].value))
            our_curve.append(float(m_our["train/ce_loss"].value))
            ref_aux.append(float(m_ref["train/lb_loss"].value))
            our_aux.append(float(m_our["train/lb_loss"].value))
    finally:
        CUDAMoEBackend.aux_to_tokens = before
    gaps = [abs(a - b) for a, b in zip(ref_curve, our_curve)]
    return {
        "model": {k: model_kw[k] for k in ("n_layers", "d_model", "num_experts", "top_k", "vocab_size", "max_seq_len")},
        "batch": batch, "steps": steps, "lr": lr,
        "reference_ce": ref_curve, "ours_ce": our_curve, "reference_lb": ref_aux, "ours_lb": our_aux,
        "step0_gap": gaps[0], "max_gap": max(gaps),
        "max_rel_gap": max(g / max(abs(a), 1e-6) for g, a in zip(gaps, ref_curve)),
        "reference_drop": ref_curve[0] - ref_curve[-1], "ours_drop": our_curve[0] - our_curve[-1],
    }
