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


q_ints = st.lists(st.integers(-2**31, 2**31 - 1), min_size=0, max_size=40)


@FAST
@given(st.integers(0, 2**62), st.lists(st.tuples(st.integers(0, 500), st.one_of(st.none(), q_ints), q_ints), max_size=8, unique_by=lambda t: t[0]),
       st.floats(0.0, 10.0, width=32))
def test_checkpoint_bytes_roundtrip_and_any_damage_is_noticed(step, layers, gamma):
    c = C.NangilaCheckpoint()
    c.step = step
    c.predictor_step = step
    c.quantizer_gamma = gamma
    for lid, prev, cur in layers:
        c.set_layer(lid, prev, cur)
    c.seal()
    raw = c.to_bytes()
    back = C.NangilaCheckpoint.from_bytes(raw)
    assert back.verify_integrity() and back.to_bytes() == raw and back.step == step
    assert back.layer_ids() == sorted(lid for lid, _, _ in layers)
    for lid, prev, cur in layers:
        assert back.get_layer(lid) == (prev if prev else None if prev is None else prev, cur) or back.get_layer(lid) == (prev, cur)
    if layers and any(cur for _, _, cur in layers):
        lid, prev, cur = next(t for t in layers if t[2])
        back.set_layer(lid, prev, [cur[0] ^ 1] + cur[1:])
        assert not back.verify_integrity()


@settings(max_examples=int(os.environ.get("NANGILA_PROPERTY_EXAMPLES", "25")), deadline=None, derandomize="NANGILA_PROPERTY_EXAMPLES" not in os.environ)
@given(st.integers(2, 6), st.integers(2, 12), st.integers(8, 40), st.integers(0, 2**31), st.floats(0.5, 0.99))
def test_sculptor_masks_are_always_valid_and_passengers_hang_on_drivers(n_layers, width, steps, seed, threshold):
    rng = np.random.default_rng(seed)
    s = nangila.Sculptor(float(threshold))
    base = rng.normal(size=(steps, width))
    gains = rng.uniform(0.2, 3.0, size=n_layers)
    independent = rng.random(n_layers) < 0.4
    for t in range(steps):
        for lid in range(n_layers):
            g = rng.normal(size=width) if independent[lid] else gains[lid] * base[t] + 0.01 * rng.normal(size=width)
            s.record(lid, g.astype(np.float32))
        s.end_step()
    mask = C.TopologyMask.from_bytes(s.generate_mask())
    mask.validate()
    assert mask.num_layers() == n_layers and mask.num_drivers() >= 1
    assert mask.num_drivers() + mask.num_passengers() == n_layers
    drivers = set(mask.drivers())
    for lid, driver, alpha, beta in mask.passengers():
        assert driver in drivers and mask.is_passenger(lid) and not mask.is_driver(lid) and lid not in drivers
        assert np.isfinite(alpha) and np.isfinite(beta)
        if threshold >= 0.9 and steps * width >= 200:
            assert not independent[lid]   # with enough samples and a high bar, noise is not tied to a driver
    assert C.TopologyMask.from_bytes(mask.to_bytes()).to_bytes() == mask.to_bytes()


@FAST
@given(st.lists(st.floats(0.125, 10.0, width=32), min_size=5, max_size=120), st.integers(1, 10), st.floats(0.01, 0.5), st.integers(1, 4))
def test_safe_mode_only_compresses_when_active_and_counts_every_check(losses, interval, threshold, max_fail):
    sm = C.SafeMode(C.SafeModeConfig(check_interval=interval, divergence_threshold=float(threshold), max_consecutive_failures=max_fail))
    checks = 0
    for step, loss in enumerate(losses):
        if sm.should_check(step):
            action = sm.check(step, float(loss))
            checks += 1
            assert action in (C.SafeModeAction.Continue, C.SafeModeAction.TriggerFallback, C.SafeModeAction.RecoveryComplete,
                              C.SafeModeAction.NoCheck, C.SafeModeAction.CanaryTest)
        state = sm.state()
        assert sm.should_compress() == (state == C.SafeModeState.Active) or state == C.SafeModeState.Recovering
    sm.force_fallback()
    assert sm.state() == C.SafeModeState.Fallback and not sm.should_compress()
    sm.reset()
    assert sm.state() == C.SafeModeState.Active and sm.should_compress()
