"""Unit tests of the C++ core through its Python bindings. The numeric expectations are the ones
the reference embeds in its own unit tests (nangila-core/src/*.rs `#[cfg(test)]` modules)."""
import math
import struct

import numpy as np
import pytest

import nangila
from nangila import _C as C


def f32(*v):
    return np.array(v, dtype=np.float32)


# ---- config -------------------------------------------------------------------------------------
def test_config_defaults_and_presets():
    c = nangila.NangilaConfig()
    assert (c.momentum, c.warmup_steps, c.shadow_run_steps, c.quantize_bits) == (pytest.approx(0.9), 1000, 100, 4)
    assert c.threshold == pytest.approx(0.95) and c.dgc_sparsity == pytest.approx(0.999) and c.power_sgd_rank == 1
    assert c.compressor_type == nangila.CompressorType.PredictionResidual == 0
    cons, aggr = nangila.NangilaConfig.conservative(), nangila.NangilaConfig.aggressive()
    assert cons.threshold == pytest.approx(0.97) and cons.dgc_sparsity == pytest.approx(0.99) and cons.power_sgd_rank == 2
    assert cons.monitor_interval == 500 and aggr.threshold == pytest.approx(0.90)


def test_config_validation():
    nangila.NangilaConfig(momentum=0.9, threshold=0.95, warmup_steps=1000, shadow_run_steps=100, quantize_bits=4)
    with pytest.raises(ValueError):
        nangila.NangilaConfig(momentum=1.5)
    with pytest.raises(ValueError):
        nangila.NangilaConfig(quantize_bits=16)
    with pytest.raises(ValueError):
        nangila.NangilaConfig(power_sgd_rank=0)
    with pytest.raises(ValueError):
        nangila.NangilaConfig(dgc_sparsity=1.5)


def test_config_kwargs_of_reference_smoke_test():
    c = nangila.NangilaConfig(momentum=0.9, threshold=0.95, warmup_steps=10, shadow_run_steps=5, quantize_bits=4,
                              compressor_type=nangila.CompressorType.DGC, dgc_sparsity=0.99, power_sgd_rank=2)
    assert c.compressor_type == 1 and c.warmup_steps == 10


# ---- SyncMode -------------------------------------------------------------------------------------
def test_sync_mode():
    assert (nangila.SyncMode.ASYNC, nangila.SyncMode.ALWAYS, nangila.SyncMode.PERIODIC) == (0, 1, 2)
    assert repr(nangila.SyncMode(0)) == "SyncMode.ASYNC"
    assert repr(nangila.SyncMode(1)) == "SyncMode.ALWAYS"
    assert repr(nangila.SyncMode(2)) == "SyncMode.PERIODIC"
    for bad in (-1, 3, 100):
        with pytest.raises(ValueError, match="Invalid sync mode"):
            nangila.SyncMode(bad)


# ---- Q8.23 ----------------------------------------------------------------------------------------
def test_q823_roundtrip_and_arithmetic():
    for v in [0.0, 1.0, -1.0, 0.5, -0.5, 0.9, 127.5, -128.0]:
        assert abs(C.q8_23_to_f32(C.q8_23_from_f32(v)) - v) < 1.2e-7
    q = C.q8_23_from_f32
    assert abs(C.q8_23_to_f32(C.q8_23_add(q(1.5), q(2.5))) - 4.0) < 1e-6
    assert abs(C.q8_23_to_f32(C.q8_23_sub(q(5.0), q(3.0))) - 2.0) < 1e-6
    assert abs(C.q8_23_to_f32(C.q8_23_mul(q(2.0), q(3.0))) - 6.0) < 1e-6
    # g_hat = g_t + mu (g_t - g_{t-1}) = 1.18
    pred = C.q8_23_add(q(1.0), C.q8_23_mul(C.q8_23_sub(q(1.0), q(0.8)), q(0.9)))
    assert abs(C.q8_23_to_f32(pred) - 1.18) < 1e-5
    assert abs(C.q8_23_to_f32(C.q8_23_fma(q(1.0), q(0.2), q(0.9))) - 1.18) < 1e-5


def test_q823_saturation_and_clamp():
    q = C.q8_23_from_f32
    assert C.q8_23_to_f32(C.q8_23_add(q(255.0), q(10.0))) > 200.0  # saturates, does not wrap
    assert q(1e9) == 2**31 - 1 and q(-1e9) == -(2**31)
    assert q(float("nan")) == 0
    assert q(-256.0) == -(2**31)
    n0 = C.q8_23_saturation_count()
    q(300.0)
    assert C.q8_23_saturation_count() == n0 + 1


def test_fixed_buffer_hash_is_deterministic():
    x = np.sin(np.arange(1000, dtype=np.float32) * 0.001)
    assert C.fixed_buffer_hash(x) == C.fixed_buffer_hash(x.copy())
    y = x.copy()
    y[17] += 1e-3
    assert C.fixed_buffer_hash(x) != C.fixed_buffer_hash(y)


def test_siphash_vectors():
    # official SipHash-2-4 test vector (key 00..0f, message 00..0e)
    k0 = int.from_bytes(bytes(range(8)), "little")
    k1 = int.from_bytes(bytes(range(8, 16)), "little")
    assert C.siphash24(bytes(range(15)), k0, k1) == 0xA129CA6149BE45E5
    # streaming splits do not change the result; 1-3 differs from 2-4
    assert C.siphash13(b"abcdefghijklmnop") != C.siphash24(b"abcdefghijklmnop")
    # a u32 written after a u64 equals the 12 concatenated bytes
    p = C.Predictor(0.9, 0)
    h0 = p.state_hash()
    assert h0 == C.siphash13(struct.pack("<Q", 0))


# ---- dtype ----------------------------------------------------------------------------------------
def test_dtype_roundtrips():
    x = f32(0.0, 1.0, -2.5, 3.14159, 65504.0, 1e-5, -1e-7)
    h = C.f16_bytes_to_f32(C.f32_to_f16_bytes(x))
    assert np.allclose(h, x.astype(np.float16).astype(np.float32), rtol=0, atol=0)
    import torch

    b = C.bf16_bytes_to_f32(C.f32_to_bf16_bytes(x))
    want = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(b, want)


# ---- predictor ------------------------------------------------------------------------------------
def test_predictor_momentum_prediction():
    p = C.Predictor(0.9, 0)
    p.update(0, f32(1.0, 2.0, 3.0))
    p.update(0, f32(1.1, 2.1, 3.1))
    assert np.allclose(p.predict(0), [1.19, 2.19, 3.19], atol=1e-3)


def test_predictor_history_warmup_hash_force_sync():
    p = C.Predictor(0.9, 0)
    p.update(0, f32(1.0, 2.0))
    assert not p.can_predict(0)
    with pytest.raises(RuntimeError):
        p.predict(0)
    w = C.Predictor(0.9, 100)
    for _ in range(99):
        w.step()
    assert not w.is_ready()
    w.step()
    assert w.is_ready()
    a, b = C.Predictor(0.9, 0), C.Predictor(0.9, 0)
    for i in range(10):
        g = f32(i * 0.1, i * 0.2)
        a.update(0, g)
        b.update(0, g)
    assert a.state_hash() == b.state_hash()
    b.update(0, f32(9.0, 9.0))
    assert a.state_hash() != b.state_hash()
    f = C.Predictor(0.9, 0)
    f.force_sync_layer(0, f32(1.0, 2.0, 3.0))
    assert f.can_predict(0) and abs(f.predict(0)[0] - 1.0) < 1e-3
    assert np.allclose(f.predict_partial(0, 1, 3), [2.0, 3.0], atol=1e-3)


def test_predictor_snapshots_and_adaptive_momentum():
    p = C.Predictor(0.9, 0)
    p.update(3, f32(0.5, -0.25))
    p.update(3, f32(0.75, 0.0))
    snap = p.export_snapshots()
    assert snap[3][0] == [C.q8_23_from_f32(0.5), C.q8_23_from_f32(-0.25)]
    q = C.Predictor(0.9, 0)
    q.restore_snapshots(snap)
    assert np.array_equal(q.predict(3), p.predict(3))
    for e in [1.0, 1.0, 1.0, 2.0, 2.0, 2.0]:  # rising error -> more conservative momentum
        p.record_error(3, e)
    assert p.get_momentum(3) < 0.9
    assert p.get_momentum(99) == pytest.approx(0.9)


def test_predictor_memory_mode():
    p = C.Predictor(0.9, 0)
    p.set_large_model_threshold(1 << 20)
    p.update(0, np.zeros(3 << 20, np.float32))
    p.step()
    mode, total, layers, _mb = p.memory_stats()
    assert mode == C.MemoryMode.DriversOnly and total == 3 << 20 and layers == 1
    p.set_driver_layers([5])
    assert p.should_track_layer(5) and not p.should_track_layer(0)


# ---- quantizer ------------------------------------------------------------------------------------
def test_pack_unpack_int4():
    v = [1, -2, 3, -4, 5, -6, 7, -8]
    packed = C.pack_int4(v)
    assert len(packed) == 4 and packed[0] == (1 | (0xE << 4))
    assert C.unpack_int4(packed, len(v)) == v
    assert C.unpack_int4(C.pack_int4([3, -1, 2]), 3) == [3, -1, 2]


def test_quantize_roundtrip_and_ratio():
    q = C.Quantizer.int4()
    q.set_gamma(0.1)
    q.set_dynamic_gamma(False)
    x = f32(0.1, 0.2, -0.3, 0.5, -0.7)
    c = q.quantize(x, 0, 0)
    assert np.all(np.abs(q.dequantize(c) - x) < 0.15)
    big = C.Quantizer.int4().quantize(np.full(1000, 0.1, np.float32), 0, 0)
    assert big.compression_ratio(1000) > 6.0
    assert np.allclose(q.dequantize_partial(c, 1, 4), q.dequantize(c)[1:4])


def test_quantizer_unbiased_for_negative_values_and_reference_mode_is_not():
    x = np.full(20000, -0.25, np.float32)  # -2.5 levels at gamma 0.1
    q = C.Quantizer(4, False)
    q.set_gamma(0.1)
    assert abs(q.dequantize(q.quantize(x, 1, 7)).mean() + 0.25) < 2e-3
    r = C.Quantizer(4, False, True)  # reference_exact: rounds negatives away from zero with p = frac
    r.set_gamma(0.1)
    assert abs(r.dequantize(r.quantize(x, 1, 7)).mean() + 0.25) < 2e-3  # frac = 0.5 is the symmetric case
    x2 = np.full(20000, -0.23, np.float32)  # -2.3 levels: frac 0.7
    assert abs(q.dequantize(q.quantize(x2, 1, 7)).mean() + 0.23) < 2e-3
    assert abs(r.dequantize(r.quantize(x2, 1, 7)).mean() + 0.23) > 0.02


def test_quantizer_reference_gamma_is_lagging_ema():
    r = C.Quantizer(4, True, True)
    r.quantize(np.full(100, 0.07, np.float32), 0, 0)
    assert r.gamma() == pytest.approx(0.99 * 1.0 + 0.01 * 0.01, rel=1e-4)
    q = C.Quantizer(4, True)
    q.quantize(np.full(100, 0.07, np.float32), 0, 0)
    assert q.gamma() == pytest.approx(0.01, rel=1e-4)


def test_quantizer_offset_determinism_and_nan():
    x = np.random.default_rng(0).normal(size=64).astype(np.float32)
    q1, q2 = C.Quantizer(4, False), C.Quantizer(4, False)
    for q in (q1, q2):
        q.set_gamma(0.3)
    full = q1.unpack(q1.quantize(x, 2, 5))
    shard = q2.unpack(q2.quantize(x[32:], 2, 5, 32))
    assert shard == full[32:]
    y = x.copy()
    y[3] = np.nan
    y[4] = np.inf
    d = q1.dequantize(q1.quantize(y, 0, 0))
    assert d[3] == 0.0 and d[4] == 0.0


# ---- packets --------------------------------------------------------------------------------------
def test_packet_header_roundtrip_and_flags():
    h = C.PacketHeader.new_driver(12345, 42)
    raw = h.to_bytes()
    assert len(raw) == 32 and raw[:2] == b"\x47\x4e" and raw[2] == 1 and raw[3] == 0x02
    assert struct.unpack_from("<I", raw, 4)[0] == 12345 and struct.unpack_from("<I", raw, 8)[0] == 42
    assert C.PacketHeader.from_bytes(raw) == h
    fs = C.PacketHeader.new_force_sync(500, 10)
    assert fs.is_force_sync() and fs.is_driver() and fs.flags == 0x03
    ps = C.PacketHeader.new_passenger(500, 10)
    assert ps.is_passenger() and not ps.is_driver()
    pr = C.PacketHeader.new_partial_retransmit(1, 2, 100, 200)
    assert pr.is_partial_retransmit() and (pr.start_offset, pr.end_offset) == (100, 200)
    assert C.PacketHeader.from_bytes(b"short") is None


def test_packet_crc():
    assert C.crc32(b"123456789") == 0xCBF43926
    p = C.Packet(C.PacketHeader.new_driver(100, 5), bytes([1, 2, 3, 4, 5, 6, 7, 8]))
    assert p.verify()
    raw = bytearray(p.to_bytes())
    raw[32 + 3] ^= 0xFF
    assert not C.Packet.from_bytes(bytes(raw)).verify()
    assert C.Packet.from_bytes(p.to_bytes()).verify()


# ---- mask -----------------------------------------------------------------------------------------
def test_mask_roles_ratio_roundtrip():
    m = C.TopologyMask()
    m.add_driver(0)
    m.add_driver(1)
    m.add_passenger(2, 0, 0.95, 0.01)
    m.add_passenger(3, 1, 0.87, 0.02)
    assert (m.num_drivers(), m.num_passengers()) == (2, 2)
    assert m.is_driver(0) and m.is_passenger(3)
    raw = m.to_bytes()
    assert struct.unpack_from("<I", raw, 0)[0] == 4 and len(raw) == 4 + 2 * 5 + 2 * 17
    back = C.TopologyMask.from_bytes(raw)
    assert back.get_role(2)[0] == "passenger" and back.get_role(2)[1] == 0
    assert back.get_role(2)[2] == pytest.approx(0.95)
    one = C.TopologyMask()
    one.add_driver(0)
    for i in range(1, 10):
        one.add_passenger(i, 0, 0.9, 0.0)
    assert one.compression_ratio() == pytest.approx(10.0)
    assert one.fsdp_ordered_layers()[0] == 0 and one.prefetch_hints()[0] == (0, 0)
    assert one.dependencies_ready(3, {0}) and not one.dependencies_ready(3, set())


def test_mask_accepts_any_entry_order_and_rejects_bad_tag():
    raw = struct.pack("<I", 2) + struct.pack("<IBIff", 7, 1, 3, 0.5, 0.25) + struct.pack("<IB", 3, 0)
    m = C.TopologyMask.from_bytes(raw)
    assert m.is_driver(3) and m.get_role(7) == ("passenger", 3, 0.5, 0.25)
    with pytest.raises(RuntimeError):
        C.TopologyMask.from_bytes(struct.pack("<IIB", 1, 0, 9))
    with pytest.raises(IOError):
        C.TopologyMask.from_bytes(struct.pack("<II", 1, 0))


def test_mask_validation():
    ok = C.TopologyMask()
    ok.add_driver(0)
    ok.add_driver(1)
    ok.add_passenger(2, 0, 0.9, 0.0)
    ok.validate()
    bad = C.TopologyMask()
    bad.add_driver(0)
    bad.add_passenger(1, 99, 0.9, 0.0)
    with pytest.raises(RuntimeError, match="non-existent"):
        bad.validate()
    pp = C.TopologyMask()
    pp.add_driver(0)
    pp.add_passenger(1, 0, 0.9, 0.0)
    pp.add_passenger(2, 1, 0.8, 0.0)
    with pytest.raises(RuntimeError, match="non-driver"):
        pp.validate()
    chk = C.TopologyMask()
    chk.add_driver(0)
    chk.add_passenger_checked(1, 0, 0.9, 0.0)
    for args in [(2, 99, 0.8, 0.0), (3, 3, 0.7, 0.0), (4, 1, 0.6, 0.0)]:
        with pytest.raises(RuntimeError):
            chk.add_passenger_checked(*args)
    chk.promote_to_driver(1)
    assert chk.is_driver(1) and chk.num_passengers() == 0


# ---- compressors ----------------------------------------------------------------------------------
def _cfg(**kw):
    return nangila.NangilaConfig(warmup_steps=0, shadow_run_steps=0, **kw)


def test_dgc_top_k_and_accumulation():
    c = C.HostCompressor(_cfg(compressor_type=1, dgc_sparsity=0.6))
    out = c.decompress(c.compress(f32(1.0, 5.0, 2.0, 4.0, 3.0), 0), 0)
    assert list(out) == [0.0, 5.0, 0.0, 4.0, 0.0]
    d = C.HostCompressor(_cfg(compressor_type=1, dgc_sparsity=0.99))
    assert d.decompress(d.compress(f32(1.0, 0, 0, 0, 0), 0), 0)[0] == 1.0
    assert d.decompress(d.compress(f32(0.1, 2.0, 0, 0, 0), 0), 0)[1] == 2.0
    assert d.decompress(d.compress(f32(0.3, 0, 0, 0, 0), 0), 0)[0] == pytest.approx(0.4, abs=1e-6)
    assert C.dgc_keep_count(1000, 0.999) == 1 and C.dgc_keep_count(5, 0.6) == 2


def test_dgc_momentum_correction():
    d = C.HostCompressor(_cfg(compressor_type=1, dgc_sparsity=0.5), dgc_momentum=0.5)
    # u = g, v = g -> sends index 1; then u,v zeroed there
    assert list(d.decompress(d.compress(f32(1.0, 2.0), 0), 0)) == [0.0, 2.0]
    # index 0: u = 0.5*1 + 1 = 1.5, v = 1 + 1.5 = 2.5 ; index 1: u = 0.1, v = 0.1
    assert list(d.decompress(d.compress(f32(1.0, 0.1), 0), 0)) == [2.5, 0.0]


def test_power_sgd_orthogonalize_and_rank1_exact():
    m = C.orthogonalize_columns(np.array([[1.0, 1.0], [0.0, 1.0]], np.float32))
    assert abs(float(m[:, 0] @ m[:, 1])) < 1e-6
    assert abs(float(m[:, 0] @ m[:, 0]) - 1.0) < 1e-6 and abs(float(m[:, 1] @ m[:, 1]) - 1.0) < 1e-6
    c = C.HostCompressor(_cfg(compressor_type=2, power_sgd_rank=1))
    g = np.array([[1.0, 1.0], [0.0, 0.0]], np.float32)
    rec = c.decompress(c.compress(g, 0), 0)
    assert np.allclose(rec, g.reshape(-1), atol=1e-5)
    q0 = C.powersgd_initial_q(6, 2)
    assert np.allclose(q0.T @ q0, np.eye(2), atol=1e-5)


def test_power_sgd_error_feedback_converges():
    rng = np.random.default_rng(0)
    g = (rng.normal(size=(16, 3)) @ rng.normal(size=(3, 12))).astype(np.float32)  # rank 3
    c = C.HostCompressor(_cfg(compressor_type=2, power_sgd_rank=3))
    errs = []
    for _ in range(4):
        rec = c.decompress(c.compress(g, 0), 0).reshape(16, 12)
        errs.append(np.linalg.norm(rec - g) / np.linalg.norm(g))
    assert errs[-1] < 0.05 < 1.0


def test_prediction_residual_pipeline_roundtrip():
    c = C.HostCompressor(_cfg())
    rng = np.random.default_rng(1)
    base = rng.normal(size=512).astype(np.float32) * 0.1
    for t in range(2):
        c.update(0, base * (1 + 0.1 * t))
        c.step()
    g = base * 1.2 + rng.normal(size=512).astype(np.float32) * 0.002
    pkt = c.compress(g, 0)
    assert len(pkt) < 512 * 4 / 6
    rec = c.decompress(pkt, 0)
    assert np.linalg.norm(rec - g) / np.linalg.norm(g) < 0.02
    assert c.last_prediction_error() < 0.2 and c.quantizer_gamma() > 0
    assert c.name() == "prediction_residual"


# ---- reconstructor / state / hook -----------------------------------------------------------------
def _mask_bytes(drivers, passengers=()):
    m = C.TopologyMask()
    for d in drivers:
        m.add_driver(d)
    for p in passengers:
        m.add_passenger(*p)
    return m.to_bytes()


def test_hook_creation_and_warmup_passthrough_is_exact():
    h = nangila.NangilaHook.all_drivers(10)
    assert not h.is_compression_enabled() and h.current_step() == 0
    g = f32(1.0, 2.0, 3.0, 4.0)
    pkt = h.compress(0, g)
    assert pkt[3] == 0  # passthrough flags
    assert np.array_equal(h.decompress(0, pkt), g)
    st = h.get_stats()
    assert set(st) == {"step", "compression_enabled", "num_drivers", "num_passengers",
                       "mask_compression_ratio", "quantizer_gamma"}
    assert st["num_drivers"] == 10


def test_hook_compresses_after_warmup_and_telemetry():
    cfg = nangila.NangilaConfig(warmup_steps=2, shadow_run_steps=2)
    h = nangila.NangilaHook(_mask_bytes([0]), cfg)
    for i in range(5):
        g = f32(1.0 + i * 0.1, 2.0, 3.0)
        h.compress(0, g)
        h.update(0, g)
        h.step()
    assert h.is_compression_enabled()
    pkt = h.compress(0, f32(1.5, 2.0, 3.0))
    assert pkt[3] & 0x02  # driver
    rec = h.decompress_gathered(0, pkt)
    assert rec.shape == (3,) and np.allclose(rec, [1.5, 2.0, 3.0], atol=0.3)
    t = h.get_layer_telemetry(0)
    assert set(t) == {"total_original_bytes", "total_compressed_bytes", "compression_count", "avg_compression_ratio",
                      "min_compression_ratio", "max_compression_ratio", "avg_prediction_error", "passenger_skip_count"}
    assert t["compression_count"] == 2 and t["total_original_bytes"] == 24  # step 4 and this call
    assert h.get_layer_telemetry(55) is None
    s = h.get_summary_telemetry()
    assert s["total_compressions"] == 2 and s["num_layers_tracked"] == 1


def test_hook_passenger_is_synthesised_from_driver():
    cfg = nangila.NangilaConfig(warmup_steps=0, shadow_run_steps=0)
    h = nangila.NangilaHook(_mask_bytes([0], [(1, 0, 0.5, 0.25)]), cfg)
    h.step()
    g = np.linspace(-1, 1, 128).astype(np.float32)
    drv = h.decompress_gathered(0, h.compress(0, g))
    ppk = h.compress(1, g * 0.5 + 0.25)
    assert len(ppk) == 32 and ppk[3] == 0x04  # empty passenger packet
    pas = h.decompress_gathered(1, ppk)
    assert np.allclose(pas, 0.5 * drv + 0.25, atol=1e-6)
    assert h.get_layer_telemetry(1)["passenger_skip_count"] == 1


def test_hook_crc_failure_recovery_and_force_sync():
    cfg = nangila.NangilaConfig(warmup_steps=0, shadow_run_steps=0)
    tx = nangila.NangilaHook(_mask_bytes([0]), cfg)
    rx = nangila.NangilaHook(_mask_bytes([0]), cfg)
    rx.set_partial_retransmit(False)
    tx.step(); rx.step()
    g = np.linspace(0, 1, 64).astype(np.float32)
    for i in range(3):
        bad = bytearray(tx.compress(0, g))
        bad[40] ^= 0xFF
        rx.decompress(0, bytes(bad))
        assert rx.crc_failure_count(0) == (i + 1) % 3
    assert rx.recovery_mode(0) == C.RecoveryMode.Pending
    # the side that detected the problem sends a FORCE_SYNC packet next: full FP32, flags 0x03
    pkt = rx.compress(0, g)
    assert pkt[3] == 0x03 and rx.recovery_mode(0) == C.RecoveryMode.Active
    out = tx.decompress_gathered(0, pkt)
    assert np.array_equal(out, g)
    rx.update(0, g)
    assert rx.recovery_mode(0) == C.RecoveryMode.Normal
    # stale packets are rejected by the point-to-point receive path
    tx2 = nangila.NangilaHook(_mask_bytes([0]), cfg)
    p_old = tx2.compress(0, g)
    tx2.step()
    p_new = tx2.compress(0, g)
    rx2 = nangila.NangilaHook(_mask_bytes([0]), cfg)
    rx2.decompress(0, p_new)
    assert rx2.decompress(0, p_old).shape[0] in (1, 64)  # falls back to history / zeros, no exception


def test_hook_hash_verification_and_safe_mode():
    h = nangila.NangilaHook.all_drivers(4)
    assert not h.should_verify_hash()
    h.set_hash_verify_interval(2)
    h.step(); h.step()
    assert h.should_verify_hash()
    assert h.verify_hash(h.predictor_hash())
    assert not h.verify_hash(h.predictor_hash() ^ 1)
    assert h.recovery_mode(0) == C.RecoveryMode.Pending
    cfg = nangila.NangilaConfig(warmup_steps=0, shadow_run_steps=0)
    s = nangila.NangilaHook(_mask_bytes([0]), cfg)
    s.enable_safe_mode(C.SafeModeConfig(check_interval=1, divergence_threshold=0.05, max_consecutive_failures=2))
    assert s.report_validation_loss(1.0) == C.SafeModeAction.NoCheck  # step 0
    for _ in range(10):
        s.step()
        s.report_validation_loss(1.0)
    assert s.is_compression_enabled()
    for _ in range(5):
        s.step()
        s.report_validation_loss(1.5)
    assert s.is_paused() and not s.is_compression_enabled()
    g = f32(1.0, 2.0)
    assert s.compress(0, g)[3] == 0  # passthrough while paused


def test_hook_from_mask_file(tmp_path):
    path = tmp_path / "mask.bin"
    path.write_bytes(_mask_bytes([0, 1], [(2, 0, 0.9, 0.0)]))
    h = nangila.NangilaHook.from_mask_file(str(path))
    assert h.get_stats()["num_passengers"] == 1
    assert h.get_stats()["mask_compression_ratio"] == pytest.approx(1.5)
    with pytest.raises(IOError):
        nangila.NangilaHook.from_mask_file(str(tmp_path / "missing.bin"))


# ---- safe mode ------------------------------------------------------------------------------------
def test_safe_mode_state_machine():
    s = C.SafeMode(C.SafeModeConfig())
    for i in (100, 200, 300):
        s.check(i, 1.0)
    assert s.stats()["baseline_loss"] is not None
    d = C.SafeMode(C.SafeModeConfig(divergence_threshold=0.05, max_consecutive_failures=2))
    for i in range(10):
        d.check(i * 100, 1.0)
    for i in range(10, 15):
        d.check(i * 100, 1.5)
    assert not d.should_compress()
    r = C.SafeMode(C.SafeModeConfig(check_interval=50, divergence_threshold=0.05, max_consecutive_failures=1,
                                    recovery_cooldown=100, canary_fraction=0.1, canary_steps=50, canary_max_failures=1))
    for i in range(10):
        r.check(i * 50, 1.0)
    for i in range(10, 15):
        r.check(i * 50, 1.5)
    assert r.state() == C.SafeModeState.Fallback
    for i in range(15, 40):
        r.check(i * 50, 1.0)
    assert r.state() in (C.SafeModeState.Recovering, C.SafeModeState.Active)
    f = C.SafeMode(C.SafeModeConfig(divergence_threshold=0.05, max_consecutive_failures=3))
    for i in range(10):
        f.check(i * 100, 1.0)
    f.check(1000, 1.5)
    f.check(1100, 1.5)
    assert f.stats()["failure_count"] > 0
    for i in range(12, 40):
        f.check(i * 100, 1.0)
    assert f.stats()["failure_count"] == 0
    c = C.SafeMode(C.SafeModeConfig(check_interval=10, canary_steps=20))
    c.enter_canary()
    assert c.state() == C.SafeModeState.Canary and not c.should_compress()
    assert c.check(10, 1.0) == C.SafeModeAction.CanaryTest
    assert c.check(20, 1.0) == C.SafeModeAction.RecoveryComplete and c.should_compress()
    p = C.SafeModeConfig.conservative()
    assert (p.check_interval, p.max_consecutive_failures, p.recovery_cooldown) == (50, 2, 1000)
    assert C.SafeModeConfig.relaxed().divergence_threshold == pytest.approx(0.01)


# ---- sculptor -------------------------------------------------------------------------------------
def test_sculptor_detects_correlation_and_builds_mask():
    s = nangila.Sculptor(0.9)
    for step in range(100):
        b = step * 0.1
        s.record(0, f32(b, b * 2, b * 3))
        s.record(1, f32(b * 0.5, b, b * 1.5))
        s.end_step()
    assert s.correlation(0, 1) > 0.95
    a, beta = s.coupling(0, 1)
    assert a == pytest.approx(0.5, abs=1e-3) and abs(beta) < 1e-3
    m = nangila.Sculptor(0.95)
    for step in range(50):
        b = math.sin(step)
        m.record(0, f32(b, b * 2))
        m.record(1, f32(b * 0.8, b * 1.6))
        m.record(2, f32(math.cos(step), float(step)))
        m.end_step()
    mask = C.TopologyMask.from_bytes(m.generate_mask())
    assert mask.num_layers() == 3 and mask.num_drivers() >= 1 and mask.num_passengers() >= 1
    assert m.num_samples() == 50 and m.num_layers() == 3
    mask.validate()
    m.reset()
    assert m.num_layers() == 0


def test_sculptor_auto_end_step_and_errors():
    s = nangila.Sculptor()
    with pytest.raises(RuntimeError):
        s.generate_mask()
    for step in range(20):  # no explicit end_step: a repeated layer id closes the step
        b = float(step)
        s.record(0, f32(b, -b))
        s.record(1, f32(2 * b, -2 * b))
    assert s.num_steps() == 19
    mask = C.TopologyMask.from_bytes(s.generate_mask())
    assert mask.num_passengers() == 1
    # layers of different sizes never pair
    d = nangila.Sculptor()
    for step in range(10):
        d.record(0, f32(step, step))
        d.record(1, f32(step, step, step))
        d.end_step()
    assert d.correlation(0, 1) is None
    assert C.TopologyMask.from_bytes(d.generate_mask()).num_passengers() == 0


def test_sculptor_strategies_schedule_pairs():
    s = nangila.Sculptor()
    for i in range(6):
        s.record(i, np.full(4, float(i + 1), np.float32))
    assert len(s.scheduled_pairs(list(range(6)))) == 15
    s.set_sampling_strategy("knn", 2)
    assert 0 < len(s.scheduled_pairs(list(range(6)))) <= 12
    s.set_sampling_strategy("hierarchical", 3)
    assert len(s.scheduled_pairs(list(range(6)))) > 0
    s.set_sampling_strategy("random", 2)
    assert len(s.scheduled_pairs(list(range(6)))) <= 12
    big = C.Sculptor.new_large_model(0.95, 600)
    assert big.threshold() == pytest.approx(0.95)


# ---- metrics / report / checkpoint ------------------------------------------------------------------
def test_metrics_prometheus_and_json():
    m = C.MetricsCollector()
    m.record_step(True)
    m.record_step(False)
    m.record_bytes(1000, 100)
    m.record_fallback()
    snap = m.snapshot()
    assert snap["compression_ratio"] == pytest.approx(10.0) and snap["bytes_saved"] == 900
    assert snap["steps_total"] == 2 and snap["steps_compressed"] == 1 and snap["fallback_count"] == 1
    text = m.to_prometheus()
    for name in ["nangila_compression_ratio", "nangila_virtual_throughput_gbps", "nangila_physical_throughput_gbps",
                 "nangila_steps_total", "nangila_steps_compressed", "nangila_bytes_received",
                 "nangila_bytes_transmitted", "nangila_bytes_saved", "nangila_fallback_total", "nangila_uptime_seconds"]:
        assert f"# TYPE {name}" in text
    assert "nangila_compression_ratio 10.000" in text
    import json

    assert json.loads(m.to_json())["bytes_received"] == 1000


def test_topology_report_json():
    import json

    m = C.TopologyMask()
    m.add_driver(0)
    m.add_passenger(1, 0, 0.5, 0.1)
    rep = json.loads(m.report_json())
    assert rep["summary"] == {"num_layers": 2, "num_drivers": 1, "num_passengers": 1,
                              "compression_ratio": 2.0, "threshold": pytest.approx(0.95)}
    assert rep["layers"][1]["role"] == "passenger" and rep["layers"][0]["source_id"] is None
    assert rep["dependency_graph"][0]["relationship"] == "drives" and rep["correlation_matrix"] is None
    json.loads(m.report_json(False))


def test_checkpoint_format_and_hash(tmp_path):
    c = C.NangilaCheckpoint()
    c.step = 100
    c.predictor_step = 100
    c.quantizer_gamma = 0.1
    c.set_layer(0, [1, 2, 3], [4, 5, 6])
    c.set_layer(5, None, [7])
    assert c.compute_hash() == c.compute_hash()
    c.seal()
    raw = c.to_bytes()
    assert raw[:8] == b"NZCHK001" and struct.unpack_from("<I", raw, 8)[0] == 1
    assert struct.unpack_from("<Q", raw, 12)[0] == 100
    # hash = SipHash-1-3 over step, then (id, prev..., current...) per ascending layer
    stream = struct.pack("<Q", 100) + struct.pack("<I", 0) + struct.pack("<6i", 1, 2, 3, 4, 5, 6) + \
        struct.pack("<I", 5) + struct.pack("<i", 7)
    assert c.state_hash == C.siphash13(stream)
    path = str(tmp_path / "c.nzchk")
    c.save(path)
    back = C.NangilaCheckpoint.load(path)
    assert back.verify_integrity() and back.get_layer(5) == (None, [7]) and back.layer_ids() == [0, 5]
    back.set_layer(0, [1, 2, 3], [4, 5, 99])
    assert not back.verify_integrity()
    with pytest.raises(RuntimeError):
        C.NangilaCheckpoint.from_bytes(b"BADMAGIC" + raw[8:])
    c.add_extra("predres.ef", 0, f32(0.5, 0.25))
    v2 = C.NangilaCheckpoint.from_bytes(c.to_bytes())
    assert v2.version == 2 and v2.extra_sections()[0][0] == "predres.ef"


def test_hook_checkpoint_roundtrip(tmp_path):
    cfg = nangila.NangilaConfig(warmup_steps=0, shadow_run_steps=0)
    h = nangila.NangilaHook(_mask_bytes([0]), cfg)
    rng = np.random.default_rng(0)
    for _ in range(3):
        g = rng.normal(size=64).astype(np.float32)
        h.update(0, h.decompress_gathered(0, h.compress(0, g)))
        h.step()
    path = str(tmp_path / "hook.nzchk")
    h.save_checkpoint(path)
    h2 = nangila.NangilaHook(_mask_bytes([0]), cfg)
    h2.load_checkpoint(path)
    assert h2.predictor_hash() == h.predictor_hash() and h2.current_step() == 3
    g = rng.normal(size=64).astype(np.float32)
    assert h.compress(0, g) == h2.compress(0, g)


def test_gradient_history_ring():
    h = C.GradientHistory(3)
    for i in range(5):
        h.push(0, np.full(10, float(i), np.float32))
    assert h.depth(0) == 3
    assert abs(h.get(0, 0)[0] - 4.0) < 1e-3 and abs(h.get(0, 2)[0] - 2.0) < 1e-3
    h5 = C.GradientHistory(5)
    for i in range(5):
        h5.push(0, np.full(10, float(i), np.float32))
    assert abs(h5.rewind(0, 2)[0] - 2.0) < 1e-3 and h5.depth(0) == 3
    assert h5.get(7, 0) is None


def test_public_surface():
    for name in ["NangilaConfig", "NangilaHook", "Sculptor", "SyncMode", "CompressorType", "cuda_available",
                 "__version__", "NangilaDDPHook", "NangilaCppHook", "CPP_HOOK_AVAILABLE", "register_nangila_hook"]:
        assert hasattr(nangila, name), name
    assert nangila.__version__ == "0.1.0"
    assert isinstance(nangila.cuda_available(), bool)
    assert C.max_compressed_size(10) == 16 + 12 + 40 + 32
