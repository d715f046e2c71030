"""Property tests of the host core (hypothesis): statements that must hold for every input, next to the example-based
checks of ``test_core.py``. The reference has no property tests.

The committed run is derandomised (the same 60 examples every time, so that the tier cannot turn red by chance);
``NANGILA_PROPERTY_EXAMPLES=3000 pytest tests/test_core_properties.py`` explores with fresh random examples."""
import os
import zlib

import numpy as np
import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

import nangila  # noqa: E402
from nangila import _C as C  # noqa: E402

finite32 = st.floats(min_value=-1e4, max_value=1e4, allow_nan=False, allow_infinity=False, width=32)
vectors = st.lists(finite32, min_size=1, max_size=300).map(lambda v: np.asarray(v, dtype=np.float32))
FAST = settings(max_examples=int(os.environ.get("NANGILA_PROPERTY_EXAMPLES", "60")), deadline=None, derandomize="NANGILA_PROPERTY_EXAMPLES" not in os.environ)


@FAST
@given(st.binary(min_size=0, max_size=512))
def test_crc32_is_the_zlib_crc(data):
    assert C.crc32(data) == zlib.crc32(data) & 0xFFFFFFFF


@FAST
@given(st.integers(0, 2**32 - 1), st.integers(0, 2**32 - 1), st.binary(min_size=0, max_size=200), st.data())
def test_packet_roundtrip_and_any_flipped_payload_bit_is_caught(step, layer, payload, data):
    p = C.Packet(C.PacketHeader.new_driver(step, layer), payload)
    raw = p.to_bytes()
    back = C.Packet.from_bytes(raw)
    assert back.verify() and back.header.step == step and back.header.layer_id == layer and bytes(back.payload) == payload
    if payload:
        bit = data.draw(st.integers(0, 8 * len(payload) - 1))
        damaged = bytearray(raw)
        damaged[32 + bit // 8] ^= 1 << (bit % 8)
        q = C.Packet.from_bytes(bytes(damaged))
        assert q is None or not q.verify()
    # every proper prefix is either refused or fails verification
    cut = data.draw(st.integers(0, len(raw) - 1))
    q = C.Packet.from_bytes(raw[:cut])
    assert q is None or not q.verify() or cut == len(raw)


@FAST
@given(vectors, st.integers(0, 1000), st.integers(0, 10**6), st.booleans())
def test_block_quantizer_error_is_within_one_level_and_zero_stays_zero(x, layer, step, stochastic):
    q = C.Quantizer(4, True)
    q.set_stochastic(stochastic)
    c = q.quantize(x, layer, step)
    y = np.asarray(q.dequantize(c))
    assert y.shape == x.shape
    for b in range(0, len(x), 64):
        blk = x[b:b + 64]
        level = float(np.abs(blk).max()) / 7.0
        bound = level * (1.0 if stochastic else 0.5) * (1 + 1e-5) + 1e-30
        assert np.abs(y[b:b + 64] - blk).max() <= bound
    assert np.all(y[x == 0.0] == 0.0)
    # the same key gives the same bytes, another step may round differently but stays within the bound
    assert bytes(q.quantize(x, layer, step).data) == bytes(c.data)


@FAST
@given(vectors)
def test_quantizer_shards_draw_the_same_random_numbers_as_the_whole(x):
    whole, part = C.Quantizer(4, False), C.Quantizer(4, False)
    for q in (whole, part):
        q.set_gamma(max(float(np.abs(x).max()) / 7.0, 1e-6))
    cut = len(x) // 2
    full = whole.unpack(whole.quantize(x, 3, 9))
    tail = part.unpack(part.quantize(x[cut:], 3, 9, cut))
    assert list(tail) == list(full[cut:])


@FAST
@given(st.lists(st.integers(-8, 7), min_size=0, max_size=200))
def test_int4_packing_roundtrip(values):
    packed = C.pack_int4(values)
    assert len(packed) == (len(values) + 1) // 2
    assert list(C.unpack_int4(packed, len(values))) == values


@FAST
@given(st.floats(min_value=-255.0, max_value=255.0, allow_nan=False, width=32), st.floats(min_value=-255.0, max_value=255.0, allow_nan=False, width=32))
def test_q8_23_is_within_half_an_lsb_and_add_saturates(a, b):
    lsb = 2.0 ** -23
    qa, qb = C.q8_23_from_f32(a), C.q8_23_from_f32(b)
    assert abs(C.q8_23_to_f32(qa) - a) <= lsb
    s = C.q8_23_to_f32(C.q8_23_add(qa, qb))
    exact = a + b
    if -256.0 < exact < 255.99:
        assert abs(s - exact) <= 3 * lsb + abs(exact) * 2.0 ** -22
    else:
        assert abs(s) >= 255.0 and (s > 0) == (exact > 0)   # clamps toward the sign of the true sum, never wraps


@FAST
@given(st.lists(st.tuples(st.integers(0, 40), st.integers(0, 40), st.floats(0.125, 2.0, width=32), st.floats(-1.0, 1.0, width=32)), max_size=25))
def test_mask_bytes_roundtrip(edges):
    m = C.TopologyMask()
    drivers = set()
    for passenger, driver, alpha, beta in edges:
        if passenger == driver or passenger in drivers:
            continue
        if not m.is_passenger(driver):
            m.add_driver(driver)
            drivers.add(driver)
            if not m.is_driver(passenger) and not m.is_passenger(passenger):
                m.add_passenger(passenger, driver, float(alpha), float(beta))
    back = C.TopologyMask.from_bytes(m.to_bytes())
    assert back.to_bytes() == m.to_bytes()
    assert sorted(back.drivers()) == sorted(m.drivers()) and sorted(back.passengers()) == sorted(m.passengers())


@settings(max_examples=int(os.environ.get("NANGILA_PROPERTY_EXAMPLES", "25")), deadline=None, derandomize="NANGILA_PROPERTY_EXAMPLES" not in os.environ)
@given(st.lists(st.lists(finite32, min_size=8, max_size=200).map(lambda v: np.asarray(v, dtype=np.float32)), min_size=3, max_size=6), st.integers(0, 3))
def test_two_hooks_fed_the_same_stream_agree_bit_for_bit(stream, warmup):
    n = min(len(v) for v in stream)
    cfg = nangila.NangilaConfig(warmup_steps=warmup, shadow_run_steps=0)
    a, b = nangila.NangilaHook.all_drivers(1, cfg), nangila.NangilaHook.all_drivers(1, cfg)
    seen = 0.0
    for g in stream:
        g = np.ascontiguousarray(g[:n])
        seen = max(seen, float(np.abs(g).max()))
        pa, pb = a.compress(0, g), b.compress(0, g)
        assert bytes(pa) == bytes(pb)
        out = np.asarray(a.decompress(0, pa))
        assert np.array_equal(out, np.asarray(b.decompress(0, pb)))
        a.update(0, out)
        b.update(0, out)
        a.step()
        b.step()
        assert a.predictor_hash() == b.predictor_hash()
        if a.is_compression_enabled():
            # the residual g - prediction is at most (1 + 1 + momentum) times the largest gradient seen, and the
            # reconstruction is off by at most one of its seven levels
            assert np.abs(out - g).max() <= 2.9 * seen / 7.0 * 1.01 + 1e-6
