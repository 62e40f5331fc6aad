"""The symmetric heap without a GPU: the C++ host test (forked ranks over a memfd + mmap driver table) and the
Python provider on gloo ranks over a stand-in for the extension's four entry points."""
import shutil
import subprocess
from pathlib import Path

import pytest
import torch

from tests.conftest import run_distributed

ROOT = Path(__file__).resolve().parent.parent


def test_cpp_host_suite(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = tmp_path / "test_symmetric_heap"
    build = subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", str(ROOT / "nanotitan_b200/csrc/runtime"),
                            str(ROOT / "tests/cpp/test_symmetric_heap.cpp"), "-o", str(exe), "-lpthread"],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "ALL PASSED" in run.stdout, run.stdout + run.stderr


class _FakeExt:
    """The extension's heap entry points over host memory; records what the provider asked for."""

    def __init__(self):
        self.opened, self.freed, self.closed, self.next_alloc = [], [], [], 1

    def symm_heap_open(self, job, rank, world, device, timeout_ms):
        self.opened.append((job, rank, world, device, timeout_ms))
        self.world = world
        return 7

    def symm_heap_alloc(self, heap, nbytes, multicast):
        assert heap == 7 and multicast
        raw = torch.zeros(nbytes, dtype=torch.uint8)
        alloc_id, self.next_alloc = self.next_alloc, self.next_alloc + 1
        return raw, [1000 * alloc_id + r for r in range(self.world)], 5000 + alloc_id, alloc_id

    def symm_heap_free(self, heap, alloc_id):
        self.freed.append(alloc_id)

    def symm_heap_close(self, heap):
        self.closed.append(heap)


def _provider_rank(rank, world):
    import torch.distributed as dist

    from nanotitan_b200.parallel.symm_memory import NativeSymmetricMemory

    ext = _FakeExt()
    mem = NativeSymmetricMemory(None, torch.device("cpu"), ext=ext)
    (job, r, w, device, timeout_ms), = ext.opened
    assert (r, w, device, timeout_ms) == (rank, world, 0, 60000)
    jobs = [None] * world
    dist.all_gather_object(jobs, job)
    assert len(set(jobs)) == 1 and jobs[0], "every rank must open the heap under the same job name"

    a = mem.empty(24, torch.bfloat16)
    b = mem.empty(10, torch.int32)
    assert a.dtype == torch.bfloat16 and a.numel() == 24 and b.dtype == torch.int32 and b.numel() == 10
    assert mem.peer_ptrs(a) == [1000 + r for r in range(world)] and mem.multicast_ptr(a) == 5001
    assert mem.peer_ptrs(b.view(2, 5)) == [2000 + r for r in range(world)], "views of an allocation name the same allocation"
    mem.free(a)
    assert ext.freed == [1]
    mem.close()
    assert ext.freed == [1, 2] and ext.closed == [7]


@pytest.mark.distributed
def test_native_provider_on_two_ranks():
    run_distributed(_provider_rank, 2)


def test_provider_choice(monkeypatch):
    from nanotitan_b200.parallel import symm_memory

    monkeypatch.setenv("NT_SYMM_HEAP", "torch")
    assert isinstance(symm_memory.make_provider(None, torch.device("cpu")), symm_memory.TorchSymmetricMemory)
    monkeypatch.setenv("NT_SYMM_HEAP", "nvshmem")
    with pytest.raises(ValueError, match="NT_SYMM_HEAP"):
        symm_memory.make_provider(None, torch.device("cpu"))
