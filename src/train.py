from nanotitan_b200.train import *  # noqa: F401,F403
from nanotitan_b200.train import main, parse_args, reduce_metrics  # noqa: F401

if __name__ == "__main__":
    main()
