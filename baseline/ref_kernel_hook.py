"""Baseline "compress, then call NCCL": a DDP comm hook that runs the reference's own CUDA kernels
(compiled unmodified by ``build_ref_kernels.py``) in the data flow of the reference's GPU-native hook
(python/nangila/ddp.py:236-284): predict-subtract-quantize kernel, all-gather of the sizes with a host
read, all-gather of the padded INT4 bytes, one dequantize-reconstruct kernel per rank, stack + mean,
copy back, history rotation.

The Rust state machine that normally sits between the hook and the kernels (packet header, CRC,
predictor-hash check, gamma bookkeeping) cannot be built here (no Rust toolchain), so this file keeps
only what that layer contributes to the data path: FP32 history buffers per bucket and a single
quantization step ``gamma`` per bucket taken from the previous step's residual (max |r| / 7, one host
read per bucket and step). It is a measuring stick for the fused kernels, not a reimplementation of the
reference's API.
"""
import ctypes
import os
from typing import Dict

import torch
import torch.distributed as dist

_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libnangila_ref_kernels.so")
        if not os.path.exists(path):
            raise RuntimeError("baseline/_ref/libnangila_ref_kernels.so is missing: run baseline/build_ref_kernels.py")
        lib = ctypes.CDLL(path)
        vp, f, i = ctypes.c_void_p, ctypes.c_float, ctypes.c_int
        lib.launch_predict_subtract_quantize.argtypes = [vp, vp, vp, f, f, vp, i, vp, i, ctypes.c_uint64, ctypes.c_uint32]
        lib.launch_predict_subtract_quantize.restype = i
        lib.launch_dequantize_add_reconstruct.argtypes = [vp, vp, vp, f, f, vp, i, vp, i]
        lib.launch_dequantize_add_reconstruct.restype = i
        _LIB = lib
    return _LIB


class RefKernelHook:
    def __init__(self, process_group=None, warmup_steps: int = 100, momentum: float = 0.9, sync_mode: int = 0):
        self.group = process_group
        self.world = dist.get_world_size(process_group)
        self.warmup_steps = warmup_steps
        self.momentum = momentum
        self.sync_mode = sync_mode
        self.step_count = 0
        self.state: Dict[int, dict] = {}
        self.kernel_launches = 0
        self.__name__ = self.__qualname__ = "ref_kernel_hook"

    def step(self) -> None:
        self.step_count += 1

    def fast_forward(self, to_step: int) -> None:
        self.step_count = max(self.step_count, to_step)

    # the surface bench.py expects of a hook
    def get_kernel_launches(self) -> int:
        return self.kernel_launches

    def _check_device_status(self) -> None:
        torch.cuda.synchronize()

    def get_stats(self) -> dict:
        return {"overall_compression_ratio": 8.0 if self.step_count >= self.warmup_steps else 1.0,
                "compression_enabled": self.step_count >= self.warmup_steps, "kernel_launches": self.kernel_launches}

    def _state(self, index: int, n: int, dev) -> dict:
        st = self.state.get(index)
        if st is None or st["n"] != n:
            z = lambda: torch.zeros(n, dtype=torch.float32, device=dev)  # noqa: E731
            st = self.state[index] = {"n": n, "prev": z(), "curr": z(), "gamma": None}
        return st

    def __call__(self, state, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
        tensor = bucket.buffer()
        index = int(bucket.index())
        n = tensor.numel()
        st = self._state(index, n, tensor.device)
        fut: torch.futures.Future = torch.futures.Future()
        if self.step_count < self.warmup_steps:
            dist.all_reduce(tensor, group=self.group)
            tensor.div_(self.world)
            st["prev"], st["curr"] = st["curr"], st["prev"]
            st["curr"].copy_(tensor)
            fut.set_result(tensor)
            return fut
        lib = _lib()
        stream = ctypes.c_void_p(torch.cuda.current_stream(tensor.device).cuda_stream)
        g32 = tensor.float().contiguous()
        pred = st["curr"] + self.momentum * (st["curr"] - st["prev"])
        if st["gamma"] is None:
            st["gamma"] = (g32 - pred).abs().amax() / 7.0
        gamma = max(float(st["gamma"].item()), 1e-12)  # host read, as the reference's size exchange has
        packed = torch.empty((n + 1) // 2, dtype=torch.uint8, device=tensor.device)
        err = lib.launch_predict_subtract_quantize(g32.data_ptr(), st["curr"].data_ptr(), st["prev"].data_ptr(), self.momentum,
                                                   gamma, packed.data_ptr(), n, stream, self.sync_mode, self.step_count, index)
        assert err == 0, f"reference predict kernel: cuda error {err}"
        size = torch.tensor([packed.numel()], dtype=torch.long, device=tensor.device)
        sizes = [torch.empty_like(size) for _ in range(self.world)]
        dist.all_gather(sizes, size, group=self.group)
        max_size = max(int(s.item()) for s in sizes)
        gathered = [torch.empty(max_size, dtype=torch.uint8, device=tensor.device) for _ in range(self.world)]
        gam = torch.tensor([gamma], dtype=torch.float32, device=tensor.device)
        gammas = [torch.empty_like(gam) for _ in range(self.world)]
        dist.all_gather(gathered, packed, group=self.group)
        dist.all_gather(gammas, gam, group=self.group)
        outs = []
        for r in range(self.world):
            out = torch.empty(n, dtype=torch.float32, device=tensor.device)
            err = lib.launch_dequantize_add_reconstruct(gathered[r].data_ptr(), st["curr"].data_ptr(), st["prev"].data_ptr(),
                                                        self.momentum, float(gammas[r].item()), out.data_ptr(), n, stream,
                                                        self.sync_mode)
            assert err == 0, f"reference reconstruct kernel: cuda error {err}"
            outs.append(out)
        self.kernel_launches += 1 + self.world
        averaged = torch.stack(outs, dim=0).mean(dim=0)
        st["gamma"] = (g32 - pred).abs().amax() / 7.0  # next step's quantization step (lagging by one step)
        tensor.copy_(averaged)
        st["prev"], st["curr"] = st["curr"], st["prev"]
        st["curr"].copy_(averaged)
        fut.set_result(tensor)
        return fut
