"""GPU methods of :class:`nangila.NangilaHook`: ``compress_gpu``, ``decompress_gpu``, ``update_gpu``.

Same names and signatures as the reference (nangila-hook/src/python.rs:315-460), where they were
placeholders that returned uninitialised tensors. Here they run the host core's prediction-residual
compressor on the device (``csrc/kernels/packet_codec.cu``) and produce / consume the host's own packet
format, so a packet made by ``compress_gpu`` decodes with ``decompress`` on a CPU-only peer and a packet
made by ``compress`` decodes with ``decompress_gpu``:

* ``compress_gpu(layer_id, gradient, sync_mode=2)`` returns a ``uint8`` CUDA tensor holding the whole
  packet (32-byte header with the payload's CRC32, then the payload). During warm-up the packet carries
  the raw FP32 values, as the host path does.
* ``decompress_gpu(layer_id, compressed, output_size, sync_mode=2)`` returns the FP32 CUDA tensor.
* ``update_gpu(layer_id, gradient, sync_mode=2)`` rotates the layer's two-step history on the device
  (call it with the averaged gradient after the all-reduce, as ``update`` on the host).

The history (two FP32 tensors per layer) and the error memory live on the device, attached to the hook
object; the host-side state machine supplies step numbers, warm-up and momentum. Nothing synchronises
unless ``sync_mode`` says so: 0 (ASYNC) never, 1 (ALWAYS) after every call, 2 (PERIODIC) every 100th call.
``decompress_gpu`` reads the 44 fixed bytes of the packet on the host (a small synchronising copy) to
validate it before anything is launched, and verifies the checksum unless ``sync_mode`` is 0.
"""
from __future__ import annotations

import struct
from typing import Dict, Optional

import torch

from ._C import NangilaHook

_HEADER = 32
_MAGIC, _VERSION = 0x4E47, 1
_FLAG_FORCE_SYNC, _FLAG_DRIVER, _FLAG_NO_PREDICTION = 0x01, 0x02, 0x80


def _glue():
    from .parallel.predres_engine import _glue as g

    return g()


class _LayerState:
    __slots__ = ("n", "curr", "prev", "ef", "updates")

    def __init__(self, n: int, device: torch.device):
        self.n = n
        self.curr = torch.zeros(n, dtype=torch.float32, device=device)
        self.prev = torch.zeros(n, dtype=torch.float32, device=device)
        self.ef = torch.zeros(n, dtype=torch.float32, device=device)
        self.updates = 0


def _state(hook) -> dict:
    st = hook.__dict__.get("_gpu")
    if st is None:
        st = hook.__dict__["_gpu"] = {"layers": {}, "calls": 0}
    return st


def _layer(hook, layer_id: int, n: int, device: torch.device) -> _LayerState:
    layers: Dict[int, _LayerState] = _state(hook)["layers"]
    ls = layers.get(layer_id)
    if ls is None or ls.n != n or ls.curr.device != device:
        ls = layers[layer_id] = _LayerState(n, device)
    return ls


def _maybe_sync(hook, sync_mode: int) -> None:
    st = _state(hook)
    st["calls"] += 1
    if sync_mode == 1 or (sync_mode == 2 and st["calls"] % 100 == 0):
        torch.cuda.current_stream().synchronize()


def _header_bytes(flags: int, step: int, layer_id: int, predictor_hash: int = 0) -> bytes:
    # magic u16 | version u8 | flags u8 | step u32 | layer u32 | crc u32 | hash u64 | start u32 | end u32
    return struct.pack("<HBBIIIQII", _MAGIC, _VERSION, flags, step & 0xFFFFFFFF, layer_id, 0, predictor_hash, 0, 0)


def _finish_packet(packet: torch.Tensor) -> torch.Tensor:
    """CRC32 of the payload, computed on the device, written into bytes 12..16 of the header."""
    crc = _glue().crc32(packet[_HEADER:])
    packet[12:16] = crc.view(torch.uint8)[:4]
    return packet


def compress_gpu(self: NangilaHook, layer_id: int, gradient: torch.Tensor, sync_mode: int = 2) -> torch.Tensor:
    if not (isinstance(gradient, torch.Tensor) and gradient.is_cuda):
        raise RuntimeError(f"compress_gpu requires a CUDA tensor, got {getattr(gradient, 'device', type(gradient))}")
    if gradient.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise TypeError(f"compress_gpu: unsupported dtype {gradient.dtype}")
    g = gradient.detach().contiguous().view(-1)
    n = g.numel()
    if n == 0:
        raise ValueError("compress_gpu: empty gradient")
    dev = g.device
    step = int(self.current_step())
    with torch.cuda.device(dev):
        if not self.is_compression_enabled():
            # warm-up: raw values, flags 0 (what the host's pass-through packet looks like)
            head = _header_bytes(0, step, layer_id) + struct.pack("<III", n, 1, n)
            packet = torch.empty(len(head) + 4 * n, dtype=torch.uint8, device=dev)
            packet[:len(head)] = torch.frombuffer(bytearray(head), dtype=torch.uint8).to(dev, non_blocking=True)
            packet[len(head):].view(torch.float32).copy_(g)
            out = _finish_packet(packet)
        else:
            glue = _glue()
            ls = _layer(self, layer_id, n, dev)
            have_history = ls.updates >= 2
            nbytes = int(glue.packet_payload_bytes(n))
            packet = torch.empty(_HEADER + nbytes, dtype=torch.uint8, device=dev)
            head = _header_bytes(_FLAG_DRIVER, step, layer_id)
            packet[:_HEADER] = torch.frombuffer(bytearray(head), dtype=torch.uint8).to(dev, non_blocking=True)
            glue.packet_encode(g, ls.curr if have_history else None, ls.prev if have_history else None, ls.ef,
                               float(self.momentum()), -1.0, packet[_HEADER:])
            out = _finish_packet(packet)
            self.record_external(layer_id, n * g.element_size(), _HEADER + nbytes, 0.0)
    _maybe_sync(self, sync_mode)
    return out


def decompress_gpu(self: NangilaHook, layer_id: int, compressed: torch.Tensor, output_size: int, sync_mode: int = 2) -> torch.Tensor:
    if not (isinstance(compressed, torch.Tensor) and compressed.is_cuda and compressed.dtype == torch.uint8):
        raise RuntimeError("decompress_gpu requires a uint8 CUDA tensor")
    packet = compressed.contiguous().view(-1)
    if packet.numel() < _HEADER + 8:
        raise RuntimeError(f"decompress_gpu: packet of {packet.numel()} bytes is too small")
    dev = packet.device
    fixed = bytes(packet[:min(packet.numel(), _HEADER + 12)].cpu().numpy())
    magic, version, flags, _step, layer, crc, _hash, _s, _e = struct.unpack("<HBBIIIQII", fixed[:_HEADER])
    if magic != _MAGIC or version != _VERSION:
        raise RuntimeError("decompress_gpu: not a nangila packet (bad magic or version)")
    if layer != layer_id:
        raise RuntimeError(f"decompress_gpu: packet is for layer {layer}, expected {layer_id}")
    with torch.cuda.device(dev):
        glue = _glue()
        if sync_mode != 0:
            got = int(glue.crc32(packet[_HEADER:]).item()) & 0xFFFFFFFF
            if got != crc:
                raise RuntimeError(f"decompress_gpu: checksum mismatch on layer {layer_id} ({got:#x} != {crc:#x})")
        out = torch.empty(int(output_size), dtype=torch.float32, device=dev)
        if not flags & _FLAG_DRIVER:
            # raw tensor payload: u32 numel, u32 ndim, u32 dims[ndim], f32 data
            numel, ndim = struct.unpack("<II", fixed[_HEADER:_HEADER + 8])
            if numel != output_size:
                raise RuntimeError(f"decompress_gpu: packet holds {numel} elements, expected {output_size}")
            start = _HEADER + 8 + 4 * ndim
            out.copy_(packet[start:start + 4 * numel].view(torch.float32))
            if flags & _FLAG_FORCE_SYNC:
                ls = _layer(self, layer_id, numel, dev)
                ls.prev.copy_(out)
                ls.curr.copy_(out)
                ls.ef.zero_()
                ls.updates = max(ls.updates, 2)
        else:
            neg_block, numel, ndim = struct.unpack("<fII", fixed[_HEADER:_HEADER + 12])
            if neg_block != -64.0:
                raise RuntimeError("decompress_gpu: only block-64 payloads can be decoded on the device")
            if numel != output_size:
                raise RuntimeError(f"decompress_gpu: packet holds {numel} elements, expected {output_size}")
            ls = _layer(self, layer_id, numel, dev)
            use_pred = not (flags & _FLAG_NO_PREDICTION) and ls.updates >= 2
            glue.packet_decode(packet[_HEADER:], int(ndim), ls.curr if use_pred else None, ls.prev if use_pred else None,
                               float(self.momentum()), -1.0 if use_pred else 0.0, out)
    _maybe_sync(self, sync_mode)
    return out


def update_gpu(self: NangilaHook, layer_id: int, gradient: torch.Tensor, sync_mode: int = 2) -> None:
    if not (isinstance(gradient, torch.Tensor) and gradient.is_cuda):
        raise RuntimeError("update_gpu requires a CUDA tensor")
    g = gradient.detach().contiguous().view(-1)
    ls = _layer(self, layer_id, g.numel(), g.device)
    ls.prev, ls.curr = ls.curr, ls.prev   # pointer swap: the oldest buffer receives the newest gradient
    ls.curr.copy_(g)
    ls.updates += 1
    _maybe_sync(self, sync_mode)


def gpu_history(self: NangilaHook, layer_id: int) -> Optional[tuple]:
    """``(previous, current)`` FP32 device tensors of a layer, or ``None`` (tests, checkpointing)."""
    ls = _state(self)["layers"].get(layer_id)
    return None if ls is None else (ls.prev, ls.curr)


def install() -> None:
    """Attach the methods to the compiled class (instances keep their device state in ``__dict__``)."""
    NangilaHook.compress_gpu = compress_gpu
    NangilaHook.decompress_gpu = decompress_gpu
    NangilaHook.update_gpu = update_gpu
    NangilaHook.gpu_history = gpu_history
