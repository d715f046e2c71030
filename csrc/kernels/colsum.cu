// Column sums of a row-major [R, C] bf16 matrix, optionally of the elementwise product with a second
// matrix of the same shape: out_sum[c] = sum_r a[r, c], out_prod[c] = sum_r a[r, c] * b[r, c].
//
// These are the bias gradient of a linear layer (a = dY) and the weight / bias gradients of a
// LayerNorm's affine part (a = dY, b = x_hat). PyTorch's kernels for them took 72 us (LayerNorm
// gamma / beta backward) and 24 us (bias reduction) per call on [8192, 768] in the GPT-2 benchmark
// step, a quarter of the step's kernel time; a streaming read of that input is 2-4 us.
// Two stages, both with a fixed summation order (no atomics): kSplits partial sums per column, then
// one thread per column adds them. The reference ships no model code; no counterpart there.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "nangila_kernels.h"

namespace {

constexpr int kSplits = 32;   // row ranges summed independently
constexpr int kRowLanes = 8;  // threadIdx.y
constexpr int kColLanes = 32;  // threadIdx.x, four columns each

__device__ __forceinline__ void unpack4(const uint2& u, float (&f)[4]) {
    f[0] = __uint_as_float(u.x << 16);
    f[1] = __uint_as_float(u.x & 0xffff0000u);
    f[2] = __uint_as_float(u.y << 16);
    f[3] = __uint_as_float(u.y & 0xffff0000u);
}

template <bool PROD>
__global__ void __launch_bounds__(kRowLanes* kColLanes) colsum_partial_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                                                              float* __restrict__ partial, int64_t R, int C, int64_t rows_per_split) {
    __shared__ float sm[kRowLanes][kColLanes * 4];
    const int col = (blockIdx.x * kColLanes + threadIdx.x) * 4;
    const int64_t r0 = int64_t(blockIdx.y) * rows_per_split;
    const int64_t r1 = r0 + rows_per_split < R ? r0 + rows_per_split : R;
    float s[4] = {0.f, 0.f, 0.f, 0.f}, p[4] = {0.f, 0.f, 0.f, 0.f};
    if (col < C) {
        for (int64_t r = r0 + threadIdx.y; r < r1; r += kRowLanes) {
            float fa[4];
            unpack4(__ldg(reinterpret_cast<const uint2*>(a + r * C + col)), fa);
#pragma unroll
            for (int k = 0; k < 4; ++k) s[k] += fa[k];
            if (PROD) {
                float fb[4];
                unpack4(__ldg(reinterpret_cast<const uint2*>(b + r * C + col)), fb);
#pragma unroll
                for (int k = 0; k < 4; ++k) p[k] = fmaf(fa[k], fb[k], p[k]);
            }
        }
    }
#pragma unroll
    for (int pass = 0; pass < (PROD ? 2 : 1); ++pass) {
        const float* v = pass == 0 ? s : p;
#pragma unroll
        for (int k = 0; k < 4; ++k) sm[threadIdx.y][threadIdx.x * 4 + k] = v[k];
        __syncthreads();
        if (threadIdx.y == 0 && col < C) {
            float* out = partial + (int64_t(pass) * kSplits + blockIdx.y) * C + col;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float t = 0.f;
#pragma unroll
                for (int y = 0; y < kRowLanes; ++y) t += sm[y][threadIdx.x * 4 + k];
                out[k] = t;
            }
        }
        __syncthreads();
    }
}

__global__ void colsum_final_kernel(const float* __restrict__ partial, int C, int outputs, float* __restrict__ out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    for (int o = 0; o < outputs; ++o) {
        float t = 0.f;
        for (int sidx = 0; sidx < kSplits; ++sidx) t += partial[(int64_t(o) * kSplits + sidx) * C + c];
        out[int64_t(o) * C + c] = t;
    }
}

}  // namespace

extern "C" int64_t nangila_colsum_scratch_floats(int C) { return int64_t(2) * kSplits * C; }

// a, b: [R, C] bf16, C a multiple of 4, 8-byte aligned; b may be null (then only the sums are produced).
// out: [C] floats (sums), followed by [C] floats (products) when b is given. scratch: nangila_colsum_scratch_floats(C) floats.
extern "C" int nangila_colsum(const void* a, const void* b, int64_t R, int C, float* scratch, float* out, cudaStream_t stream) {
    if (!a || !scratch || !out || R <= 0 || C <= 0 || (C & 3) || (reinterpret_cast<uintptr_t>(a) & 7) || (b && (reinterpret_cast<uintptr_t>(b) & 7)))
        return int(cudaErrorInvalidValue);
    const int64_t rows_per_split = (R + kSplits - 1) / kSplits;
    dim3 grid(unsigned((C / 4 + kColLanes - 1) / kColLanes), kSplits), block(kColLanes, kRowLanes);
    if (b)
        colsum_partial_kernel<true><<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), scratch, R, C,
                                                                rows_per_split);
    else
        colsum_partial_kernel<false><<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16*>(a), nullptr, scratch, R, C, rows_per_split);
    colsum_final_kernel<<<(C + 255) / 256, 256, 0, stream>>>(scratch, C, b ? 2 : 1, out);
    return int(cudaGetLastError());
}
