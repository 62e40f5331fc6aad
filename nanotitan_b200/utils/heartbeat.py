"""Per-rank heartbeat files: host-side liveness for a supervisor or for peer ranks.

Each rank rewrites `<dir>/rank_<r>.json` after every step (atomic rename).
`stale_ranks` lists ranks whose file is missing or older than a limit.  Nothing here
touches a GPU: a lost rank is found on the host before the next collective is
launched, and the process-group timeout ends a collective that was already posted.

The reference has no failure detection (its loop only destroys the process group in a `finally`,
src/train.py:149, 224-226).
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path


class Heartbeat:
    def __init__(self, directory: str | Path, rank: int):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.rank = rank
        self.path = self.dir / f"rank_{rank}.json"

    def beat(self, step: int, **extra) -> None:
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(json.dumps({"rank": self.rank, "step": step, "time": time.time(), **extra}))
        os.replace(tmp, self.path)

    def leave(self, step: int) -> None:
        """Mark this rank as gone (clean exit or a caught failure): peers see it at their next check
        without waiting for the file to age."""
        self.beat(step, left=True)

    @staticmethod
    def read(directory: str | Path, rank: int) -> dict | None:
        path = Path(directory) / f"rank_{rank}.json"
        try:
            return json.loads(path.read_text())
        except (FileNotFoundError, json.JSONDecodeError):
            return None

    @staticmethod
    def stale_ranks(directory: str | Path, world_size: int, max_age_s: float, now: float | None = None) -> list[int]:
        now = time.time() if now is None else now
        stale = []
        for rank in range(world_size):
            rec = Heartbeat.read(directory, rank)
            if rec is None or rec.get("left") or now - rec["time"] > max_age_s:
                stale.append(rank)
        return stale


class RankFailure(RuntimeError):
    """Raised on the survivors when a peer is found dead before the next step."""


def assert_peers_alive(directory: str | Path, world_size: int, max_age_s: float) -> None:
    stale = Heartbeat.stale_ranks(directory, world_size, max_age_s)
    if stale:
        raise RankFailure(f"ranks {stale} have left or have no heartbeat newer than {max_age_s:.0f}s")
