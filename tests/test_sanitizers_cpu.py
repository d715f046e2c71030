"""Sanitizer tier (CPU): the native host code built with AddressSanitizer + UndefinedBehaviorSanitizer and driven
with hostile input. The reference has no sanitizer run at all (its CI is cargo test / pytest / rustfmt).

* ``tests/native/ffi_fuzz.cpp``: the C ABI's packet path against corrupted, truncated, over-long and random packets.
* ``nangila-node`` on a transistor-level deck, on damaged copies of it and of a partition file, and as three
  processes that exchange boundaries over TCP.
"""
import json
import os
import random
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FLAGS = ["-std=c++17", "-O0", "-g1", "-fsanitize=address,undefined", "-fno-omit-frame-pointer"]  # -O0: the compile dominates the run


def _sanitizers_available(tmp):
    if shutil.which("g++") is None:
        return False
    src = os.path.join(tmp, "probe.cpp")
    with open(src, "w") as f:
        f.write("int main() { return 0; }\n")
    r = subprocess.run(["g++", *FLAGS, "-o", os.path.join(tmp, "probe"), src], capture_output=True)
    return r.returncode == 0 and subprocess.run([os.path.join(tmp, "probe")]).returncode == 0


def _clean(stderr: str) -> bool:
    return "runtime error" not in stderr and "Sanitizer" not in stderr


@pytest.fixture(scope="module")
def built(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("san"))
    if not _sanitizers_available(tmp):
        pytest.skip("g++ with -fsanitize=address,undefined is not usable here")
    fuzz, node, tnode = os.path.join(tmp, "ffi_fuzz"), os.path.join(tmp, "nangila-node-san"), os.path.join(tmp, "nangila-node-tsan")
    jobs = [subprocess.Popen(["g++", *FLAGS, f"-I{ROOT}/csrc/core", f"-I{ROOT}/csrc/kernels", "-o", fuzz, f"{ROOT}/tests/native/ffi_fuzz.cpp",
                              f"{ROOT}/csrc/core/c_api.cpp", "-ldl", "-lpthread"], stderr=subprocess.PIPE, text=True),
            subprocess.Popen(["g++", *FLAGS, f"-I{ROOT}/csrc/spice", "-o", node, f"{ROOT}/csrc/spice/node_main.cpp", "-ldl", "-lpthread"],
                             stderr=subprocess.PIPE, text=True),
            subprocess.Popen(["g++", "-std=c++17", "-O0", "-g1", "-fsanitize=thread", f"-I{ROOT}/csrc/spice", "-o", tnode,
                              f"{ROOT}/csrc/spice/node_main.cpp", "-ldl", "-lpthread"], stderr=subprocess.PIPE, text=True)]
    for j in jobs:
        err = j.communicate(timeout=900)[1]
        assert j.returncode == 0, err[-2000:]
    return {"fuzz": fuzz, "node": node, "tsan_node": tnode, "tmp": tmp}


@pytest.mark.timeout(1200)
def test_c_abi_packet_path_under_sanitizers(built):
    r = subprocess.run([built["fuzz"], "400"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and _clean(r.stderr), (r.stdout[-500:], r.stderr[-3000:])
    accepted, rejected = (int(x) for x in r.stdout.split()[-3::2])
    assert accepted > 50 and rejected > 300   # intact packets pass, damaged ones are turned away


@pytest.mark.timeout(1200)
def test_solver_process_under_sanitizers(built):
    sys.path.insert(0, ROOT)
    import nangila_spice as ns
    from nangila_spice import correctness as cx

    tmp, node = built["tmp"], built["node"]
    case = next(c for c in cx.official_correctness_cases() if c.name == "adder2")
    deck = case.materialize(tmp)
    r = subprocess.run([node, "--partition", deck, "--tstop", "2e-10", "--dt", "1e-12", "--waveform-json", os.path.join(tmp, "w.json"),
                        "--waveform-nz", os.path.join(tmp, "w.nz")], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and _clean(r.stderr), r.stderr[-3000:]
    # three processes over TCP
    pr = ns.partition_netlist(ns.parse_netlist(deck), 3, "spectral")
    files = []
    for i, js in enumerate(pr.partition_files()):
        files.append(os.path.join(tmp, f"p{i}.json"))
        with open(files[-1], "w") as f:
            f.write(js)
    procs = [subprocess.Popen([node, "--partition", files[i], "--node-id", str(i), "-k", str(len(files)), "--rendezvous", os.path.join(tmp, "rv"),
                               "--tstop", "1e-10", "--dt", "1e-12"], stderr=subprocess.PIPE, text=True) for i in range(len(files))]
    for p in procs:
        err = p.communicate(timeout=600)[1]
        assert p.returncode == 0 and _clean(err), err[-3000:]
    # damaged inputs: any exit code, but no sanitizer report and no signal
    rng = random.Random(5)
    sources = [open(deck, "rb").read(), open(files[0], "rb").read()]
    for trial in range(40):
        data = bytearray(sources[trial % 2])
        kind = trial % 4
        if kind == 0:
            for _ in range(rng.randint(1, 6)):
                data[rng.randrange(len(data))] = rng.choice(b"0123456789-eE.,:[]{}\" \n()=*+MRCV")
        elif kind == 1:
            data = data[: rng.randrange(len(data))]
        elif kind == 2:
            i = rng.randrange(len(data) - 4)
            data[i:i + 3] = b"9e9"
        else:
            i = rng.randrange(len(data) - 4)
            data[i:i + 2] = b"-7"
        path = os.path.join(tmp, "fuzzed.sp" if trial % 2 == 0 else "fuzzed.json")
        with open(path, "wb") as f:
            f.write(data)
        r = subprocess.run([node, "--partition", path, "--tstop", "2e-11", "--dt", "1e-12"], capture_output=True, text=True, timeout=300)
        assert r.returncode >= 0 and _clean(r.stderr), (trial, r.returncode, r.stderr[-3000:])
    # decks written to strain the reader itself: arithmetic, quoting, source cards, includes
    hostile = [
        "* deep\n.param a='" + "(" * 5000 + "1" + ")" * 5000 + "'\nR1 x 0 a\nV1 x 0 1\n.end\n",
        "* unbalanced\n.param a='((1+2)' b={3*(4 c='5\nR1 x 0 'a*\nV1 x 0 {b\n.end\n",
        "* division\n.param z='1/0' n='0/0' big='1e308*1e308'\nR1 x 0 z\nR2 x 0 n\nC1 x 0 big\nV1 x 0 1\n.end\n",
        "* operators\nR1 x 0 '*'\nR2 x 0 '1**2'\nR3 x 0 '--++-1'\nR4 x 0 '1e'\nR5 x 0 '1e+'\nV1 x 0 '()'\n.end\n",
        "* sources\nV1 a 0 PWL(0)\nV2 b 0 PWL(1n 1 0 0 1n 2)\nV3 c 0 SIN()\nV4 d 0 EXP(0 1 0 0 0 0)\nV5 e 0 PWL\nI1 0 f SIN(0 1 1e30 -1 1e30 1e30)\n"
        "R1 a 0 1\nR2 b 0 1\nR3 c 0 1\nR4 d 0 1\nR5 e 0 1\nR6 f 0 1\n.end\n",
        "* includes\n.include\n.include ''\n.lib\n.lib fuzzed.sp\n.lib fuzzed.sp nosuch\n.include fuzzed.sp\n.include /\n.include /dev/null\nR1 x 0 1\nV1 x 0 1\n.end\n",
        "M",
        "X1 a b c\n",
        ".tran\n.tran x y\n.tran 0 0\n.tran -1 -1\nR1 x 0 1\nV1 x 0 1\n",
    ]
    for k, text in enumerate(hostile):
        path = os.path.join(tmp, "fuzzed.sp")
        with open(path, "w") as f:
            f.write(text)
        r = subprocess.run([node, "--partition", path, "--tstop", "2e-11", "--dt", "1e-12"], capture_output=True, text=True, timeout=300)
        assert r.returncode >= 0 and _clean(r.stderr), (k, r.returncode, r.stderr[-3000:])
    assert json.load(open(os.path.join(tmp, "w.json")))["stats"]["completed"] is True


@pytest.mark.timeout(1200)
def test_checkpoint_and_mask_tools_under_sanitizers(built, tmp_path):
    sys.path.insert(0, ROOT)
    import numpy as np

    import nangila

    tools = {}
    jobs = []
    for name in ("dump", "profile"):
        tools[name] = os.path.join(built["tmp"], f"nangila-{name}-san")
        jobs.append(subprocess.Popen(["g++", *FLAGS, f"-I{ROOT}/csrc/core", "-o", tools[name], f"{ROOT}/csrc/cli/nangila_{name}.cpp"],
                                     stderr=subprocess.PIPE, text=True))
    for j in jobs:
        err = j.communicate(timeout=900)[1]
        assert j.returncode == 0, err[-2000:]
    hook = nangila.NangilaHook.all_drivers(2, nangila.NangilaConfig(warmup_steps=0, shadow_run_steps=0))
    rng = np.random.default_rng(0)
    for _ in range(3):
        for lid in (0, 1):
            hook.update(lid, hook.decompress_gathered(lid, hook.compress(lid, rng.normal(size=32).astype(np.float32))))
        hook.step()
    ckpt = str(tmp_path / "a.ckpt")
    hook.save_checkpoint(ckpt)
    grads = tmp_path / "grads.jsonl"
    with open(grads, "w") as f:
        base = rng.normal(size=16)
        for step in range(30):
            for lid in range(3):
                f.write(json.dumps({"step": step, "layer_id": lid, "data": [float(v) for v in base * (1 + 0.1 * lid) + 0.01 * rng.normal(size=16)],
                                    "shape": [16]}) + "\n")
    mask = str(tmp_path / "mask.bin")
    r = subprocess.run([tools["profile"], "calibrate", "-g", str(grads), "-s", "20", "-t", "0.9", "-o", mask], capture_output=True, text=True)
    assert r.returncode == 0 and _clean(r.stderr), r.stderr[-2000:]
    good = {"ckpt": open(ckpt, "rb").read(), "mask": open(mask, "rb").read()}
    prng = random.Random(11)
    for trial in range(60):
        which = "ckpt" if trial % 2 == 0 else "mask"
        data = bytearray(good[which])
        kind = trial % 3
        if kind == 0:
            for _ in range(prng.randint(1, 4)):
                data[prng.randrange(len(data))] = prng.randrange(256)
        elif kind == 1:
            data = data[: prng.randrange(len(data))]
        else:
            i = prng.randrange(max(1, len(data) - 8))
            data[i:i + 8] = b"\xff" * 8   # a length field of 2^64 - 1 somewhere
        path = str(tmp_path / f"fuzzed.{which}")
        with open(path, "wb") as f:
            f.write(data)
        cmds = ([[tools["dump"], c, "-c", path] for c in ("verify", "inspect", "info")] if which == "ckpt"
                else [[tools["profile"], "info", "-m", path], [tools["profile"], "report", "-m", path, "-o", str(tmp_path / "r.json")]])
        for cmd in cmds:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=120)
            assert r.returncode >= 0 and _clean(r.stderr), (trial, cmd, r.stderr[-3000:])


@pytest.mark.timeout(1200)
def test_threaded_partitioned_run_under_thread_sanitizer(built):
    """The worker pool of the in-process partitioned run (spin-then-yield generation counter) under ThreadSanitizer."""
    sys.path.insert(0, ROOT)
    import nangila_spice as ns
    from nangila_spice import correctness as cx

    tmp = built["tmp"]
    probe = subprocess.run([built["tsan_node"], "--demo", "--tstop", "1e-11"], capture_output=True, text=True, timeout=300)
    if "FATAL: ThreadSanitizer" in probe.stderr:   # e.g. an address-space layout the runtime cannot map
        pytest.skip("ThreadSanitizer cannot run in this environment: " + probe.stderr.strip().splitlines()[0])
    case = next(c for c in cx.extended_phase1_correctness_cases() if c.name == "alu2")
    deck = case.materialize(os.path.join(tmp, "tsan"))
    pr = ns.partition_netlist(ns.parse_netlist(deck), 4, "spectral")
    files = []
    for i, js in enumerate(pr.partition_files()):
        files.append(os.path.join(tmp, "tsan", f"p{i}.json"))
        with open(files[-1], "w") as f:
            f.write(js)
    r = subprocess.run([built["tsan_node"], "--partitions", ",".join(files), "--threads", "4", "--tstop", "2e-10", "--dt", "1e-12"],
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "ThreadSanitizer" not in r.stderr and "data race" not in r.stderr, r.stderr[-3000:]
    assert "partitioned run: 200 steps" in r.stderr
