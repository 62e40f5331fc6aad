from nanotitan_b200.dist_env import *  # noqa: F401,F403
from nanotitan_b200.dist_env import barrier, cleanup, get_local_rank, get_rank, get_world_size, init_distributed, is_distributed, is_main_process  # noqa: F401
