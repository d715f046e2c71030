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
FLAGS = ["-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer"]


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
    fuzz, node = os.path.join(tmp, "ffi_fuzz"), os.path.join(tmp, "nangila-node-san")
    jobs = [subprocess.Popen(["g++", *FLAGS, f"-I{ROOT}/csrc/core", f"-I{ROOT}/csrc/kernels", "-o", fuzz, f"{ROOT}/tests/native/ffi_fuzz.cpp",
                              f"{ROOT}/csrc/core/c_api.cpp", "-ldl", "-lpthread"], stderr=subprocess.PIPE, text=True),
            subprocess.Popen(["g++", *FLAGS, f"-I{ROOT}/csrc/spice", "-o", node, f"{ROOT}/csrc/spice/node_main.cpp", "-ldl", "-lpthread"],
                             stderr=subprocess.PIPE, text=True)]
    for j in jobs:
        err = j.communicate(timeout=900)[1]
        assert j.returncode == 0, err[-2000:]
    return {"fuzz": fuzz, "node": node, "tmp": tmp}


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
    assert json.load(open(os.path.join(tmp, "w.json")))["stats"]["completed"] is True
