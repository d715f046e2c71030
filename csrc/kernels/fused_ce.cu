// Fused softmax cross-entropy over bf16 logits with a padded vocabulary (the LM head of the GPT-2
// benchmark model: 8192 rows x 50304 columns of which 50257 are classes).
//
// PyTorch's eager path slices the padded columns away, copies the logits to fp32, materialises the
// log-softmax and then the gradient: about 10 GB of traffic per step for this shape. Here the forward
// reads the bf16 logits once (online max / sum per row, one CTA per row) and the backward reads them
// once more and writes the bf16 gradient, (softmax - onehot) * g / rows, with zeros in the padded
// columns: 2.5 GB in total. The reference ships no model code, so this has no counterpart there.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "nangila_kernels.h"

namespace {

constexpr int kT = 256;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// (m, s) <- merge of two partial (max, sum of exp(x - max)) pairs
__device__ __forceinline__ void merge(float& m, float& s, float m2, float s2) {
    const float mn = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.0f : s * __expf(m - mn)) + (m2 == -INFINITY ? 0.0f : s2 * __expf(m2 - mn));
    m = mn;
}

__global__ void __launch_bounds__(kT) ce_forward_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                         float* __restrict__ losses, float* __restrict__ lse_out, int v, int64_t stride) {
    __shared__ float sm[kT / 32], ss[kT / 32];
    const int64_t row = blockIdx.x;
    const __nv_bfloat16* p = logits + row * stride;
    const int tid = threadIdx.x;
    const int v8 = v & ~7;
    float m = -INFINITY, s = 0.0f;
    for (int i = tid * 8; i < v8; i += kT * 8) {
        float f[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p + i)), f);
        float mx = f[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) mx = fmaxf(mx, f[k]);
        const float mn = fmaxf(m, mx);
        float acc = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) acc += __expf(f[k] - mn);
        s = s * __expf(m - mn) + acc;  // exp(-inf) = 0 on the first pass
        m = mn;
    }
    if (tid < v - v8) {
        const float x = __bfloat162float(p[v8 + tid]);
        merge(m, s, x, 1.0f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) merge(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
    if ((tid & 31) == 0) { sm[tid >> 5] = m; ss[tid >> 5] = s; }
    __syncthreads();
    if (tid == 0) {
        float M = sm[0], S = ss[0];
        for (int w = 1; w < kT / 32; ++w) merge(M, S, sm[w], ss[w]);
        const float lse = M + __logf(S);
        const int64_t t = targets[row];
        const float xt = (t >= 0 && t < v) ? __bfloat162float(p[t]) : lse;  // an out-of-range target contributes no loss
        lse_out[row] = lse;
        losses[row] = lse - xt;
    }
}

__global__ void __launch_bounds__(kT) ce_backward_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                          const float* __restrict__ lse, const float* __restrict__ grad_out, float inv_rows,
                                                          __nv_bfloat16* __restrict__ grad, int v, int64_t stride) {
    const int64_t row = blockIdx.x;
    const __nv_bfloat16* p = logits + row * stride;
    __nv_bfloat16* g = grad + row * stride;
    const float scale = grad_out[0] * inv_rows, l = lse[row];
    const int64_t t64 = targets[row];
    const int t = (t64 >= 0 && t64 < v) ? int(t64) : -1;
    const int cols = int(stride);
    for (int i = threadIdx.x * 8; i < cols; i += kT * 8) {
        float f[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p + i)), f);
        uint32_t out[4];
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
            float a = (i + k < v && t >= 0) ? __expf(f[k] - l) * scale : 0.0f;
            float b = (i + k + 1 < v && t >= 0) ? __expf(f[k + 1] - l) * scale : 0.0f;
            if (i + k == t) a -= scale;
            if (i + k + 1 == t) b -= scale;
            const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            out[k / 2] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(g + i) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

}  // namespace

// logits: rows x stride bf16 (stride a multiple of 8, base 16-byte aligned), classes = the first v columns.
extern "C" int nangila_ce_forward(const void* logits, const int64_t* targets, float* losses, float* lse, int64_t rows, int v, int64_t stride,
                                  cudaStream_t stream) {
    if (!logits || !targets || !losses || !lse || rows <= 0 || v <= 0 || stride < v || (stride & 7) || (reinterpret_cast<uintptr_t>(logits) & 15))
        return int(cudaErrorInvalidValue);
    if (rows > 2147483647) return int(cudaErrorInvalidValue);
    ce_forward_kernel<<<unsigned(rows), kT, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), targets, losses, lse, v, stride);
    return int(cudaGetLastError());
}

// grad = (softmax(logits[:, :v]) - onehot(targets)) * grad_out[0] / rows, zeros in columns >= v.
extern "C" int nangila_ce_backward(const void* logits, const int64_t* targets, const float* lse, const float* grad_out, void* grad, int64_t rows,
                                   int v, int64_t stride, cudaStream_t stream) {
    if (!logits || !targets || !lse || !grad_out || !grad || rows <= 0 || v <= 0 || stride < v || (stride & 7) ||
        (reinterpret_cast<uintptr_t>(logits) & 15) || (reinterpret_cast<uintptr_t>(grad) & 15))
        return int(cudaErrorInvalidValue);
    if (rows > 2147483647) return int(cudaErrorInvalidValue);
    ce_backward_kernel<<<unsigned(rows), kT, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), targets, lse, grad_out, 1.0f / float(rows),
                                                          static_cast<__nv_bfloat16*>(grad), v, stride);
    return int(cudaGetLastError());
}
