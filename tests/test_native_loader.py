"""The C++ token window loader: its host test, and batch-for-batch equality with the torch DataLoader it replaces."""
import shutil
import subprocess
from pathlib import Path

import pytest
import torch
from torch.utils.data import DataLoader, DistributedSampler

from nanotitan_b200.data.dataset import PackedTokenDataset, write_synthetic_token_file
from nanotitan_b200.ops.ext import have_ext

ROOT = Path(__file__).resolve().parent.parent


def test_cpp_host_suite(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = tmp_path / "test_token_loader"
    build = subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", str(ROOT / "nanotitan_b200/csrc/runtime"),
                            str(ROOT / "tests/cpp/test_token_loader.cpp"), "-o", str(exe), "-lpthread"],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "ALL PASSED" in run.stdout, run.stdout + run.stderr


needs_ext = pytest.mark.skipif(not have_ext(), reason="the extension is not built")


@needs_ext
@pytest.mark.parametrize("replicas,rank", [(1, 0), (3, 1)])
def test_same_batches_as_the_torch_loader(tmp_path, replicas, rank):
    from nanotitan_b200.data.native_loader import NativeTokenLoader, make_train_loader

    seq_len, batch = 16, 4
    path = write_synthetic_token_file(tmp_path / "tokens.bin", 50257, 16 * 57 + 9, seed=3)
    dataset = PackedTokenDataset(path, seq_len)

    def sampler():
        return DistributedSampler(dataset, num_replicas=replicas, rank=rank, shuffle=True, seed=0)

    torch_loader = DataLoader(dataset, batch_size=batch, sampler=sampler(), drop_last=True)
    native = make_train_loader(dataset, sampler(), batch, torch.device("cpu"), num_workers=2)
    assert isinstance(native, NativeTokenLoader) and native.num_sequences == len(dataset) == 57
    assert len(native) == len(torch_loader)
    for epoch in range(2):
        torch_loader.sampler.set_epoch(epoch)
        native.sampler.set_epoch(epoch)
        want = list(torch_loader)
        got = list(native)  # batches handed out earlier must stay intact: on CPU each one is a copy
        assert len(got) == len(want) > 0
        for (gx, gy), (wx, wy) in zip(got, want):
            assert gx.dtype == torch.int64 and torch.equal(gx, wx) and torch.equal(gy, wy)


@needs_ext
def test_leaving_an_epoch_early_and_starting_over(tmp_path):
    from nanotitan_b200.data.native_loader import NativeTokenLoader

    path = write_synthetic_token_file(tmp_path / "tokens.bin", 1000, 8 * 40 + 1, seed=4)
    dataset = PackedTokenDataset(path, 8)
    loader = NativeTokenLoader(path, 8, 2, list(range(len(dataset))), torch.device("cpu"), depth=3, threads=3)
    first = next(iter(loader))  # abandon the epoch after one batch: the workers must stop, not wait for ever
    again = [b for b in loader]
    assert len(again) == 20 and torch.equal(first[0], again[0][0])
    assert torch.equal(again[5][0][1], torch.from_numpy(dataset.tokens[11 * 8 : 12 * 8].astype("int64")))
    assert torch.equal(again[5][1][1], torch.from_numpy(dataset.tokens[11 * 8 + 1 : 12 * 8 + 1].astype("int64")))


@needs_ext
def test_a_resumed_epoch_starts_where_the_interrupted_one_stopped(tmp_path):
    from nanotitan_b200.data.native_loader import make_train_loader, skip_batches

    path = write_synthetic_token_file(tmp_path / "tokens.bin", 1000, 8 * 30 + 1, seed=5)
    dataset = PackedTokenDataset(path, 8)
    for loader in (make_train_loader(dataset, DistributedSampler(dataset, num_replicas=1, rank=0, shuffle=True, seed=1), 4,
                                     torch.device("cpu"), num_workers=1),
                   DataLoader(dataset, batch_size=4, drop_last=True,
                              sampler=DistributedSampler(dataset, num_replicas=1, rank=0, shuffle=True, seed=1))):
        loader.sampler.set_epoch(2)
        whole = list(loader)
        rest = list(skip_batches(loader, 3))
        assert len(whole) == 7 and len(rest) == 4
        for (ax, ay), (bx, by) in zip(whole[3:], rest):
            assert torch.equal(ax, bx) and torch.equal(ay, by)
        assert len(list(loader)) == 7  # the skip applies to one epoch only
        assert list(skip_batches(loader, 7)) == [] and list(skip_batches(loader, 9)) == []


@needs_ext
def test_ring_slots_handed_out_as_views_stay_valid_for_two_requests(tmp_path):
    """The GPU form of the loader yields the pinned ring slots themselves; a batch must stay intact while the next
    one is requested (its host-to-device copy may still be reading it) and its slot may be refilled only after that."""
    from nanotitan_b200.data.native_loader import NativeTokenLoader

    path = write_synthetic_token_file(tmp_path / "tokens.bin", 1000, 8 * 24 + 1, seed=6)
    dataset = PackedTokenDataset(path, 8)
    loader = NativeTokenLoader(path, 8, 2, list(range(len(dataset))), torch.device("cpu"), depth=3, threads=2, views=True)
    want = [torch.stack([dataset[2 * b][0], dataset[2 * b + 1][0]]) for b in range(12)]
    previous = None
    seen = 0
    for b, (x, _) in enumerate(loader):
        assert x.data_ptr() == loader._slots[b % 3, 0].data_ptr(), "a view of the ring, not a copy"
        assert torch.equal(x, want[b])
        if previous is not None:
            assert torch.equal(previous, want[b - 1]), "the batch before this one was overwritten too early"
        previous = x
        seen += 1
    assert seen == 12
