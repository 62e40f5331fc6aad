"""`python scripts/sweep.py <sweep.toml> [--dry-run] [--log-level L]`: the reference's sweep entry path
(scripts/sweep.py:18-31).  The runner itself is `nanotitan_b200.sweep`."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from nanotitan_b200.sweep import build_runs, dump_toml, launch_command, main  # noqa: E402,F401

if __name__ == "__main__":
    raise SystemExit(main())
