"""GPU methods of NangilaHook (compress_gpu / decompress_gpu / update_gpu) and the C entry points
nangila_compress_gpu / nangila_decompress_gpu: packets made on the device decode on the host and the
other way round, against the host core as the oracle."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _hook(warmup=2, layers=4):
    import nangila

    cfg = nangila.NangilaConfig(warmup_steps=warmup, shadow_run_steps=0)
    return nangila.NangilaHook.all_drivers(layers, cfg)


def _drifting(n, steps, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    base = torch.randn(n, device="cuda", generator=g) * 0.02
    drift = torch.randn(n, device="cuda", generator=g) * 0.002
    return [base + drift * t + torch.randn(n, device="cuda", generator=g) * 2e-4 for t in range(steps)]


@pytest.mark.parametrize("n", [64 * 50, 100_003])
def test_device_packets_decode_on_the_host_and_back(n):
    dev_hook, host_hook = _hook(), _hook()
    grads = _drifting(n, 7)
    for t, g in enumerate(grads):
        g_host = g.cpu().numpy()
        pkt = dev_hook.compress_gpu(0, g, sync_mode=1)
        assert pkt.dtype == torch.uint8 and pkt.is_cuda
        # the host decodes the device's packet
        via_host = host_hook.decompress(0, bytes(pkt.cpu().numpy()))
        on_dev = dev_hook.decompress_gpu(0, pkt, n, sync_mode=1)
        assert via_host.shape[0] == n
        assert np.abs(via_host - on_dev.cpu().numpy()).max() < 2e-6, f"step {t}"
        if t < 2:
            assert np.array_equal(via_host, g_host)            # warm-up: raw FP32 values
            assert pkt.numel() == 32 + 12 + 4 * n
        else:
            assert pkt.numel() == 32 + 20 + 4 * ((n + 63) // 64) + (n + 1) // 2
            rel = np.linalg.norm(via_host - g_host) / np.linalg.norm(g_host)
            assert rel < (0.12 if t < 4 else 0.03), (t, rel)     # with two steps of history the residual is small
        # the device decodes the host's packet of the same gradient (same history on both sides)
        host_pkt = bytes(host_hook.compress(0, g_host))
        dev_dec = dev_hook.decompress_gpu(0, torch.frombuffer(bytearray(host_pkt), dtype=torch.uint8).cuda(), n)
        host_dec = _clone_decode(host_hook, host_pkt, n)
        assert np.abs(dev_dec.cpu().numpy() - host_dec).max() < 2e-6, f"step {t}"
        for h in (dev_hook, host_hook):
            h.update(0, g_host)
            h.step()
        dev_hook.update_gpu(0, g)
    prev, curr = dev_hook.gpu_history(0)
    assert torch.equal(curr, grads[-1]) and torch.equal(prev, grads[-2])


def _clone_decode(hook, pkt, n):
    """Decode with the all-gather form (no peer-step bookkeeping), so that the same hook can decode twice."""
    out = hook.decompress_gathered(0, pkt)
    assert out.shape[0] == n
    return out


def test_checksum_and_layer_are_verified():
    hook = _hook(warmup=0)
    hook.step()
    g = torch.randn(4096, device="cuda") * 0.01
    pkt = hook.compress_gpu(1, g)
    bad = pkt.clone()
    bad[100] ^= 0x10
    with pytest.raises(RuntimeError, match="checksum"):
        hook.decompress_gpu(1, bad, 4096)
    assert hook.decompress_gpu(1, bad, 4096, sync_mode=0).shape[0] == 4096   # ASYNC: no checks
    with pytest.raises(RuntimeError, match="layer"):
        hook.decompress_gpu(2, pkt, 4096)
    with pytest.raises(RuntimeError):
        hook.compress_gpu(0, torch.zeros(8))  # not a CUDA tensor


def test_error_memory_recovers_what_quantization_dropped():
    hook = _hook(warmup=0)
    hook.step()
    g = torch.randn(64 * 200, device="cuda") * 0.01
    acc = torch.zeros_like(g)
    for t in range(8):
        acc += hook.decompress_gpu(0, hook.compress_gpu(0, g), g.numel())
        hook.step()
    first = (hook.decompress_gpu(3, hook.compress_gpu(3, g), g.numel(), sync_mode=0) - g).norm()  # fresh layer: no memory yet
    assert (acc / 8 - g).norm() < 0.3 * first


def test_c_entry_points_on_device_tensors():
    from nangila import _C as C

    lib = ctypes.CDLL(C.__file__)
    vp, u32, u64, sz, i32 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_size_t, ctypes.c_int32
    lib.nangila_init_all_drivers_ex.restype = vp
    lib.nangila_init_all_drivers_ex.argtypes = [u32, u64, u64]
    lib.nangila_step.argtypes = [vp]
    lib.nangila_free.argtypes = [vp]
    lib.nangila_gpu_payload_size.restype = sz
    lib.nangila_gpu_payload_size.argtypes = [sz]
    lib.nangila_compress_gpu.argtypes = [vp, vp, vp, vp, sz, u32, vp, ctypes.POINTER(sz), vp, vp, vp, i32]
    lib.nangila_decompress_gpu.argtypes = [vp, vp, sz, vp, vp, u32, vp, sz, vp, vp, i32]
    lib.nangila_decompress.argtypes = [vp, vp, sz, u32, vp, sz]
    lib.nangila_on_complete.argtypes = [vp, vp, sz, u32]

    n = 10_000
    h = lib.nangila_init_all_drivers_ex(2, 0, 0)
    peer = lib.nangila_init_all_drivers_ex(2, 0, 0)   # a CPU-only receiver with the same history
    grads = _drifting(n, 4, seed=3)
    prev, curr = grads[0].clone(), grads[1].clone()
    for g in grads[:2]:
        a = g.cpu().numpy()
        lib.nangila_on_complete(peer, a.ctypes.data, n, 1)
    lib.nangila_step(h)
    lib.nangila_step(peer)
    g = grads[2]
    payload_bytes = lib.nangila_gpu_payload_size(n)
    packet = torch.zeros(32 + payload_bytes, dtype=torch.uint8, device="cuda")
    header = (ctypes.c_uint8 * 32)()
    scratch = torch.zeros(4, dtype=torch.int32, device="cuda")
    out_size = sz(0)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.nangila_compress_gpu(h, g.data_ptr(), curr.data_ptr(), prev.data_ptr(), n, 1, packet.data_ptr() + 32,
                                  ctypes.byref(out_size), ctypes.addressof(header), stream, scratch.data_ptr(), 2)
    assert rc == 0 and out_size.value == 32 + payload_bytes
    packet[:32] = torch.frombuffer(bytearray(bytes(header)), dtype=torch.uint8).cuda()
    out = torch.empty(n, device="cuda")
    rc = lib.nangila_decompress_gpu(h, packet.data_ptr(), packet.numel(), curr.data_ptr(), prev.data_ptr(), 1,
                                    out.data_ptr(), n, stream, scratch.data_ptr(), 1)
    assert rc == 0
    rel = ((out - g).norm() / g.norm()).item()
    assert rel < 0.03, rel
    # the same packet through the CPU entry point of a peer that holds the same history
    host_out = np.zeros(n, np.float32)
    pk = packet.cpu().numpy()
    assert lib.nangila_decompress(peer, pk.ctypes.data, pk.size, 1, host_out.ctypes.data, n) == 0
    assert np.abs(host_out - out.cpu().numpy()).max() < 2e-6
    # a damaged payload is refused before anything is launched; invalid pointers are reported
    packet[200] ^= 1
    assert lib.nangila_decompress_gpu(h, packet.data_ptr(), packet.numel(), curr.data_ptr(), prev.data_ptr(), 1,
                                      out.data_ptr(), n, stream, scratch.data_ptr(), 2) == 5
    assert lib.nangila_compress_gpu(h, None, curr.data_ptr(), prev.data_ptr(), n, 1, packet.data_ptr() + 32,
                                    ctypes.byref(out_size), ctypes.addressof(header), stream, scratch.data_ptr(), 2) == 1
    lib.nangila_free(h)
    lib.nangila_free(peer)
