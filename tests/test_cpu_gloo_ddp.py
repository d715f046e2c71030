"""CPU / gloo, world_size 2: the DDP plumbing check. fp32 MLP 784 -> 256 -> ReLU -> 10, batch 32 per
rank from N(0,1), uniform labels, cross-entropy, SGD lr 0.01, 200 steps,
register_nangila_hook(threshold=0.95, warmup_steps=100), Sculptor calibration over the first 50
steps, seed 0. Compared against plain DDP on the same data."""
import os
import socket
import sys
import warnings

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _gloo_worker import run  # noqa: E402


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(tmp_path, name, steps, use_hook, kwargs, calib=0, fixed=False):
    out = str(tmp_path / name)
    mp.spawn(run, args=(2, _port(), steps, use_hook, out, kwargs, calib, fixed), nprocs=2, join=True)
    return torch.load(out, weights_only=False), torch.load(out + ".rank0"), torch.load(out + ".rank1")


@pytest.mark.timeout(600)
def test_mlp_200_steps_with_calibration(tmp_path):
    ours, p0, p1 = _spawn(tmp_path, "ours.pt", 200, True, dict(threshold=0.95, warmup_steps=100), calib=50)
    base, _, _ = _spawn(tmp_path, "base.pt", 200, False, {})
    # warm-up is an exact average: identical losses for the first 100 steps
    assert ours["losses"][:100] == pytest.approx(base["losses"][:100], abs=1e-6)
    st = ours["stats"]
    assert st["step"] == 200 and st["compression_enabled"]
    assert st["overall_compression_ratio"] > 1.5  # 100 exact + 100 compressed (INT4) steps
    # replicas stay bit-identical under compression
    assert torch.equal(p0, p1)
    # final-loss parity with uncompressed DDP (random labels: loss stays near ln 10)
    a = sum(ours["losses"][-20:]) / 20
    b = sum(base["losses"][-20:]) / 20
    assert abs(a - b) < 0.05 * b
    # Sculptor calibration ran over 50 steps; the four parameters differ in size, so all are Drivers
    nbytes, drivers, passengers, samples = ours["mask_info"]
    assert (drivers, passengers, samples) == (4, 0, 50) and nbytes == 4 + 4 * 5
    # the metrics collector was fed by the hook: 200 steps, the second hundred compressed, bytes saved
    m = ours["metrics"]
    assert m["steps_total"] == 200 and m["steps_compressed"] == 100
    assert m["bytes_received"] > m["bytes_transmitted"] > 0 and m["bytes_saved"] == m["bytes_received"] - m["bytes_transmitted"]
    assert m["compression_ratio"] == pytest.approx(st["overall_compression_ratio"], rel=1e-3)
    assert "nangila_steps_compressed 100" in ours["prometheus"] and "# TYPE nangila_bytes_saved counter" in ours["prometheus"]


@pytest.mark.timeout(600)
def test_compressed_training_learns_fixed_batch(tmp_path):
    ours, p0, p1 = _spawn(tmp_path, "o.pt", 120, True, dict(warmup_steps=10), fixed=True)
    base, _, _ = _spawn(tmp_path, "b.pt", 120, False, {}, fixed=True)
    assert torch.equal(p0, p1)
    assert base["losses"][-1] < base["losses"][0] - 0.05
    assert abs(ours["losses"][-1] - base["losses"][-1]) < 0.05
    assert ours["stats"]["overall_compression_ratio"] > 4.0


@pytest.mark.timeout(600)
@pytest.mark.parametrize("ctype,extra", [(1, dict(dgc_sparsity=0.9)), (2, dict(power_sgd_rank=4))])
def test_dgc_and_powersgd_knobs_are_real(tmp_path, ctype, extra):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ours, p0, p1 = _spawn(tmp_path, f"c{ctype}.pt", 80, True, dict(warmup_steps=5, compressor_type=ctype, **extra),
                              fixed=True)
    base, _, _ = _spawn(tmp_path, f"b{ctype}.pt", 80, False, {}, fixed=True)
    assert torch.equal(p0, p1)
    assert ours["stats"]["overall_compression_ratio"] > 2.0
    assert ours["losses"][-1] < ours["losses"][0]  # still trains
    assert abs(ours["losses"][-1] - base["losses"][-1]) < 0.15


def test_register_rejects_non_ddp_and_warns():
    import nangila

    with pytest.raises(TypeError):
        nangila.register_nangila_hook(torch.nn.Linear(2, 2))


@pytest.mark.timeout(600)
def test_rejected_packets_fall_back_to_exact_allreduce(tmp_path):
    """Host-side fault injection: a corrupted packet seen by every rank, a truncated packet seen by one
    rank only, and a dropped packet. Each costs one exact all-reduce of that bucket; training goes on
    and the replicas stay identical."""
    faults = [dict(step=14, kind="corrupt", src=1), dict(step=18, kind="truncate", src=0, on_rank=1),
              dict(step=22, kind="drop", src=1)]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ours, p0, p1 = _spawn(tmp_path, "faulty.pt", 40, True, dict(warmup_steps=10, _faults=faults), fixed=True)
    assert ours["stats"]["recovered_failures"] == 3
    assert torch.equal(p0, p1)
    assert all(l == l for l in ours["losses"]) and ours["losses"][-1] < ours["losses"][0]
    assert ours["stats"]["compression_enabled"]


@pytest.mark.timeout(600)
def test_checkpoint_resume_continues_the_run(tmp_path):
    """Model + optimizer + hook state saved at step 15 of 30; a fresh job resumed from it ends next to
    the uninterrupted run. The first step after a resume is averaged exactly (a new DDP instance uses
    its construction-order bucket layout for one iteration, which the saved per-bucket state does not
    match), so the two trajectories differ by one step's quantization noise, not more."""
    full, f0, f1 = _spawn(tmp_path, "full.pt", 30, True, dict(warmup_steps=5, _ckpt_at=15))
    resumed, r0, r1 = _spawn(tmp_path, "resumed.pt", 30, True,
                             dict(warmup_steps=5, _resume=str(tmp_path / "full.pt.ckpt")))
    assert torch.equal(f0, f1) and torch.equal(r0, r1)
    assert (f0 - r0).abs().max().item() < 1e-4
    assert resumed["stats"]["step"] == 30 and resumed["stats"]["compression_enabled"]
    assert resumed["losses"][-1] == pytest.approx(full["losses"][-1], abs=1e-3)
    # 15 compressed steps were resumed: the byte counters keep counting from the saved values
    assert resumed["stats"]["total_original_bytes"] == full["stats"]["total_original_bytes"]


@pytest.mark.timeout(600)
@pytest.mark.parametrize("kwargs", [dict(warmup_steps=10), dict(warmup_steps=10, compressor_type=1, dgc_sparsity=0.99),
                                    dict(warmup_steps=10, compressor_type=2, power_sgd_rank=2)], ids=["predres", "dgc", "powersgd"])
def test_three_ranks_stay_identical_and_learn(tmp_path, kwargs):
    """An odd world size: the packet path gathers from two peers, and the mean divides by three."""
    out = str(tmp_path / "w3.pt")
    mp.spawn(run, args=(3, _port(), 60, True, out, kwargs, 0, True), nprocs=3, join=True)
    res = torch.load(out, weights_only=False)
    params = [torch.load(out + f".rank{i}") for i in range(3)]
    assert torch.equal(params[0], params[1]) and torch.equal(params[0], params[2])
    assert res["losses"][-1] < res["losses"][0] - 0.3 and res["stats"]["overall_compression_ratio"] > 2.0
