"""Command-line tools (exit codes 2 / 3 as in the reference) and the C ABI of the core."""
import ctypes
import glob
import json
import os
import subprocess
import sys

import numpy as np

import nangila
from nangila import _C as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(mod, *args):
    return subprocess.run([sys.executable, "-m", f"nangila.cli.{mod}", *args], cwd=ROOT, capture_output=True, text=True)


def _checkpoint(tmp_path, name, bump=0):
    cfg = nangila.NangilaConfig(warmup_steps=0, shadow_run_steps=0)
    h = nangila.NangilaHook.all_drivers(2, cfg)
    rng = np.random.default_rng(0)
    for step in range(3):
        for lid in (0, 1):
            g = rng.normal(size=32).astype(np.float32) + (bump if lid == 1 else 0)
            h.update(lid, h.decompress_gathered(lid, h.compress(lid, g)))
        h.step()
    path = str(tmp_path / name)
    h.save_checkpoint(path)
    return path


def test_dump_verify_info_inspect_diff(tmp_path):
    a = _checkpoint(tmp_path, "a.nzchk")
    b = _checkpoint(tmp_path, "b.nzchk")
    c = _checkpoint(tmp_path, "c.nzchk", bump=1.0)
    r = _run("dump", "verify", "-c", a)
    assert r.returncode == 0 and "VALID" in r.stdout
    assert "Step:" in _run("dump", "info", "-c", a).stdout
    ins = json.loads(_run("dump", "inspect", "-c", a).stdout)
    assert ins["info"]["integrity_valid"] and ins["info"]["num_layers"] == 2 and len(ins["layers"]) == 2
    same = _run("dump", "diff", "-a", a, "-b", b)
    assert same.returncode == 0 and json.loads(same.stdout)["match_status"] == "MATCH"
    diff = _run("dump", "diff", "-a", a, "-b", c)
    assert diff.returncode == 3 and json.loads(diff.stdout)["divergent_layers"] == [1]
    # flip one state byte: integrity check fails with exit code 2
    raw = bytearray(open(a, "rb").read())
    raw[48 + 4 + 1 + 4] ^= 0x01  # first history word of layer 0 (after the 48-byte header, id, flag, length)
    bad = str(tmp_path / "bad.nzchk")
    open(bad, "wb").write(bytes(raw))
    assert _run("dump", "verify", "-c", bad).returncode == 2
    assert _run("dump", "verify", "-c", str(tmp_path / "missing")).returncode == 1


def test_profile_calibrate_report_info(tmp_path):
    grads = tmp_path / "g.jsonl"
    rng = np.random.default_rng(1)
    with open(grads, "w") as f:
        for step in range(30):
            base = rng.normal(size=16)
            for lid, vec in ((0, base), (1, 0.5 * base + 0.1), (2, rng.normal(size=16))):
                f.write(json.dumps({"step": step, "layer_id": lid, "data": [float(v) for v in vec], "shape": [16]}) + "\n")
    mask = str(tmp_path / "mask.bin")
    rep = str(tmp_path / "rep.json")
    r = _run("profile", "calibrate", "-g", str(grads), "-s", "30", "-t", "0.9", "-o", mask, "--report", rep)
    assert r.returncode == 0, r.stderr
    m = C.TopologyMask.from_bytes(open(mask, "rb").read())
    assert m.num_layers() == 3 and m.num_passengers() == 1
    pid, src, alpha, beta = m.passengers()[0]
    assert {pid, src} == {0, 1}
    report = json.loads(open(rep).read())
    assert report["summary"]["num_passengers"] == 1 and report["correlation_matrix"] is not None
    info = _run("profile", "info", "-m", mask)
    assert info.returncode == 0 and "Passengers:  1" in info.stdout
    out2 = str(tmp_path / "rep2.json")
    assert _run("profile", "report", "-m", mask, "-o", out2).returncode == 0
    assert json.loads(open(out2).read())["summary"]["num_layers"] == 3
    # the mask file feeds the hook
    assert nangila.NangilaHook.from_mask_file(mask).get_stats()["num_passengers"] == 1


def test_c_abi_roundtrip_and_safe_mode(tmp_path):
    lib = ctypes.CDLL(glob.glob(os.path.join(ROOT, "nangila", "_C*.so"))[0])
    vp, u32, u64, sz = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_size_t
    lib.nangila_init_all_drivers.restype = vp
    lib.nangila_init_all_drivers.argtypes = [u32]
    lib.nangila_init_all_drivers_ex.restype = vp
    lib.nangila_init_all_drivers_ex.argtypes = [u32, u64, u64]
    lib.nangila_init.restype = vp
    lib.nangila_init.argtypes = [ctypes.c_char_p]
    lib.nangila_max_compressed_size.restype = sz
    lib.nangila_max_compressed_size.argtypes = [sz]
    lib.nangila_current_step.restype = u64
    lib.nangila_predictor_hash.restype = u64
    for fn in ("nangila_step", "nangila_is_enabled", "nangila_current_step", "nangila_predictor_hash", "nangila_free"):
        getattr(lib, fn).argtypes = [vp]
    lib.nangila_compress.argtypes = [vp, vp, sz, u32, vp, ctypes.POINTER(sz)]
    lib.nangila_decompress.argtypes = [vp, vp, sz, u32, vp, sz]
    lib.nangila_compress_ex.argtypes = [vp, vp, sz, ctypes.c_int32, u32, vp, ctypes.POINTER(sz)]
    lib.nangila_decompress_ex.argtypes = [vp, vp, sz, u32, vp, sz, ctypes.c_int32]
    lib.nangila_on_complete.argtypes = [vp, vp, sz, u32]
    lib.nangila_enable_safe_mode.argtypes = [vp, ctypes.c_float, sz, u32, sz]
    lib.nangila_report_val_loss.argtypes = [vp, ctypes.c_float]

    # warm-up: packets carry the exact FP32 values (reference test ffi.rs:476-508)
    h = lib.nangila_init_all_drivers(4)
    assert lib.nangila_is_enabled(h) == 0 and lib.nangila_current_step(h) == 0
    x = np.linspace(-1, 1, 100).astype(np.float32)
    buf = np.zeros(lib.nangila_max_compressed_size(100), np.uint8)
    n = sz(0)
    assert lib.nangila_compress(h, x.ctypes.data, 100, 0, buf.ctypes.data, ctypes.byref(n)) == 0
    out = np.zeros(100, np.float32)
    assert lib.nangila_decompress(h, buf.ctypes.data, n.value, 0, out.ctypes.data, 100) == 0
    assert np.array_equal(out, x)
    assert lib.nangila_compress(h, None, 100, 0, buf.ctypes.data, ctypes.byref(n)) == 1  # invalid pointer
    lib.nangila_free(h)

    # compression enabled from step 1; bf16 in / bf16 out
    h = lib.nangila_init_all_drivers_ex(1, 0, 0)
    lib.nangila_step(h)
    assert lib.nangila_is_enabled(h) == 1 and lib.nangila_current_step(h) == 1
    xb = C.f32_to_bf16_bytes(x)
    assert lib.nangila_compress_ex(h, xb, 100, 2, 0, buf.ctypes.data, ctypes.byref(n)) == 0
    assert n.value < 32 + 12 + 4 + 100  # INT4 + scales, far below raw FP32
    ob = ctypes.create_string_buffer(200)
    assert lib.nangila_decompress_ex(h, buf.ctypes.data, n.value, 0, ob, 100, 2) == 0
    rec = C.bf16_bytes_to_f32(ob.raw)
    assert np.abs(rec - x).max() < 0.16
    assert lib.nangila_on_complete(h, rec.ctypes.data, 100, 0) == 0
    assert lib.nangila_predictor_hash(h) != 0
    lib.nangila_enable_safe_mode(h, 0.05, 1, 2, 10)
    assert lib.nangila_report_val_loss(h, 1.0) in (0, 3)
    for _ in range(12):
        lib.nangila_step(h)
        lib.nangila_report_val_loss(h, 1.0)
    codes = []
    for _ in range(6):
        lib.nangila_step(h)
        codes.append(lib.nangila_report_val_loss(h, 2.0))
    assert 1 in codes and lib.nangila_is_enabled(h) == 0  # fallback triggered
    lib.nangila_free(h)

    mask = C.TopologyMask()
    mask.add_driver(0)
    mask.add_passenger(1, 0, 0.5, 0.0)
    path = tmp_path / "m.bin"
    path.write_bytes(mask.to_bytes())
    h = lib.nangila_init(str(path).encode())
    assert h is not None
    lib.nangila_free(h)
    assert lib.nangila_init(b"/nonexistent/mask") is None


def test_release_manifest_is_consistent():
    from nangila.cli import release_check

    assert release_check.check() == []
    assert release_check.check(tag="v0.0.0") != []
    assert release_check.main(["--tag", "v" + __import__("nangila").__version__]) == 0
