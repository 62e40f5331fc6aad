from nanotitan_b200.utils import *  # noqa: F401,F403
from nanotitan_b200.utils import load_run_config, normalize_config_arg, reduce_scalars, resolve_device, resolve_dtype, seed_everything, setup_logging, setup_tensorboard, get_profiler_trace_dir  # noqa: F401
