// Small fused kernels for the decode step around the sparse attention: what the reference's model
// file does with a dozen torch ops each (models/llama_mustafar_kernel.py:744,760 RMSNorm via the HF
// layer, :373-374 rotary embedding, :391 and :430 appending the new K/V token to the dense window,
// :761 the MLP's activation).  One token per sequence, so every tensor here is a few hundred KB: the point is
// launch count (about 60 torch kernels per layer become 4), not bandwidth.
//
// Rounding follows the torch ops they replace, step by step: fp16 tensors, every elementwise op
// computed in fp32 and rounded to fp16 once, RMS statistics in fp32.
#include "compress_common.cuh"

namespace mfar {

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
    for (int d = 16; d; d >>= 1) v += __shfl_xor_sync(kFull, v, d);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i];
    return t;
}

// x[row] (+= delta[row]);  out[row] = fp16(float(x) * rsqrt(mean(x^2) + eps)) * w
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__half* x, const __half* delta, const __half* w, __half* out,
                                                          int hidden, float eps) {
    __shared__ float red[8];
    const int64_t row = blockIdx.x;
    __half* xr = x + row * hidden;
    const __half* dr = delta ? delta + row * hidden : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < hidden; i += 256 * 8) {
        uint4 a = *reinterpret_cast<const uint4*>(xr + i);
        __half2* ah = reinterpret_cast<__half2*>(&a);
        if (dr) {
            const uint4 d = *reinterpret_cast<const uint4*>(dr + i);
            const __half2* dh = reinterpret_cast<const __half2*>(&d);
#pragma unroll
            for (int k = 0; k < 4; ++k) ah[k] = __hadd2(ah[k], dh[k]);
            *reinterpret_cast<uint4*>(xr + i) = a;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(ah[k]);
            ss += f.x * f.x + f.y * f.y;
        }
    }
    const float scale = rsqrtf(block_sum_256(ss, red) / static_cast<float>(hidden) + eps);
    __half* orow = out + row * hidden;
    for (int i = threadIdx.x * 8; i < hidden; i += 256 * 8) {
        const uint4 a = *reinterpret_cast<const uint4*>(xr + i);   // own writes: same thread, same addresses
        const uint4 g = *reinterpret_cast<const uint4*>(w + i);
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        const __half2* gh = reinterpret_cast<const __half2*>(&g);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(ah[k]);
            oh[k] = __hmul2(__floats2half2_rn(f.x * scale, f.y * scale), gh[k]);
        }
        *reinterpret_cast<uint4*>(orow + i) = o;
    }
}

// One CTA of 64 threads per (sequence, head) of the fused q|k|v projection output, head_dim 128.
// q heads: rotate, write to q_out [B*hq, 128].  k heads: rotate, write into the key window at token
// slot widx.  v heads: copy into the value window.  Rotate-half convention, cos/sin rounded to fp16
// before use, products and sums rounded to fp16 one by one (what the torch expression does).
//
// Per-step pruning (prune_rank > 0): the CTAs behind the batch * heads append CTAs prune, in place, the window token
// that has just left the group of `prune_back` most recent ones, slot widx - prune_back - 1, of every K and V window
// head: one thread pair per row, 32 rows per CTA.  It is the token the reference's torch path prunes at the end of the
// previous step (models/llama_mustafar_Kt_Mag_Vt_Mag.py:917-926, :1015-1024); this step's attention sees it pruned.
__global__ void __launch_bounds__(64) rope_append_kernel(const __half* qkv, const float* inv_freq, const int* pos_dev,
                                                         int pos_host, const int* widx_dev, int widx_host, int batch, int hq,
                                                         int hkv, __half* q_out, __half* kwin, __half* vwin, int64_t win_hs,
                                                         int64_t win_ts, int capacity, unsigned* dev_status, int prune_rank,
                                                         int prune_back) {
    const int heads = hq + 2 * hkv;
    const int widx = widx_dev ? *widx_dev : widx_host;
    if (blockIdx.x >= static_cast<unsigned>(batch) * heads) {
        const int row = (blockIdx.x - batch * heads) * 32 + (threadIdx.x >> 1), hh = threadIdx.x & 1;
        const int slot = widx - prune_back - 1;
        if (row >= 2 * batch * hkv || slot < 0 || slot >= capacity) return;   // both members of a pair leave together
        __half* win = row < batch * hkv ? kwin : vwin;
        __half* dst = win + static_cast<int64_t>(row % (batch * hkv)) * win_hs + slot * win_ts;
        uint4 v[8];
        load_prune_row(dst, hh, prune_rank, true, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) reinterpret_cast<uint4*>(dst)[2 * j + hh] = v[j];
        return;
    }
    const int b = blockIdx.x / heads, hd = blockIdx.x % heads, i = threadIdx.x;
    const __half* src = qkv + (static_cast<int64_t>(b) * heads + hd) * kD;
    const __half x1 = src[i], x2 = src[i + 64];
    // a slot outside the window (host and device counters out of step) is reported, never written
    if (hd >= hq && (widx < 0 || widx >= capacity)) {
        if (i == 0 && dev_status) atomicOr(dev_status, MFAR_DEV_BADMETA);
        return;
    }
    if (hd >= hq + hkv) {
        __half* dst = vwin + (static_cast<int64_t>(b) * hkv + (hd - hq - hkv)) * win_hs + widx * win_ts;
        dst[i] = x1;
        dst[i + 64] = x2;
        return;
    }
    const int pos = pos_dev ? *pos_dev : pos_host;
    const float ang = static_cast<float>(pos) * inv_freq[i];
    const __half c = __float2half_rn(cosf(ang)), s = __float2half_rn(sinf(ang));
    // the _rn forms keep the compiler from contracting a product and the sum into one fused multiply-add
    const __half o1 = __hsub_rn(__hmul_rn(x1, c), __hmul_rn(x2, s));
    const __half o2 = __hadd_rn(__hmul_rn(x2, c), __hmul_rn(x1, s));
    __half* dst = hd < hq ? q_out + (static_cast<int64_t>(b) * hq + hd) * kD
                          : kwin + (static_cast<int64_t>(b) * hkv + (hd - hq)) * win_hs + widx * win_ts;
    dst[i] = o1;
    dst[i + 64] = o2;
}

// out[r, j] = fp16(silu(gu[r, j])) * gu[r, width + j]
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* gu, __half* out, int64_t rows, int width) {
    const int64_t n2 = rows * (width / 2);
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; t < n2; t += static_cast<int64_t>(gridDim.x) * 256) {
        const int64_t r = t / (width / 2);
        const int j = static_cast<int>(t % (width / 2)) * 2;
        const __half2 g = *reinterpret_cast<const __half2*>(gu + r * 2 * width + j);
        const __half2 u = *reinterpret_cast<const __half2*>(gu + r * 2 * width + width + j);
        const float2 f = __half22float2(g);
        const __half2 a = __floats2half2_rn(f.x / (1.f + expf(-f.x)), f.y / (1.f + expf(-f.y)));
        *reinterpret_cast<__half2*>(out + r * width + j) = __hmul2(a, u);
    }
}

}  // namespace mfar

using namespace mfar;

extern "C" int mfar_add_rmsnorm_f16(void* x, const void* delta, const void* weight, void* out, int64_t rows, int hidden,
                                    float eps, void* stream) {
    if (rows < 0 || hidden <= 0 || (hidden % 8) != 0) return MFAR_ERR_ARG;
    if (rows == 0) return MFAR_OK;
    if (!x || !weight || !out) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(weight) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(delta) & 15))
        return MFAR_ERR_ALIGN;
    if (rows > 0x7fffffffll) return MFAR_ERR_LIMIT;
    add_rmsnorm_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__half*>(x), static_cast<const __half*>(delta), static_cast<const __half*>(weight),
        static_cast<__half*>(out), hidden, eps);
    return launch_status();
}

extern "C" int mfar_rope_append_f16(const void* qkv, const float* inv_freq, const int32_t* pos_dev, int pos,
                                    const int32_t* slot_dev, int slot, int batch, int n_q_heads, int n_kv_heads,
                                    void* q_out, void* k_window, void* v_window, int64_t win_head_stride,
                                    int64_t win_token_stride, int window_capacity, int prune_rank, int prune_back,
                                    uint32_t* dev_status, void* stream) {
    if (batch < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || pos < 0 || slot < 0 || window_capacity <= 0) return MFAR_ERR_ARG;
    if (!slot_dev && slot >= window_capacity) return MFAR_ERR_ARG;
    if (prune_rank < 0 || prune_rank > kD || prune_back < 0) return MFAR_ERR_ARG;
    if (prune_rank > 0 && ((reinterpret_cast<uintptr_t>(k_window) & 15) || (reinterpret_cast<uintptr_t>(v_window) & 15) ||
                           (win_head_stride & 7) || (win_token_stride & 7)))
        return MFAR_ERR_ALIGN;
    if (batch == 0) return MFAR_OK;
    if (!qkv || !inv_freq || !q_out || !k_window || !v_window) return MFAR_ERR_ARG;
    int64_t ctas = static_cast<int64_t>(batch) * (n_q_heads + 2 * n_kv_heads);
    if (prune_rank > 0) ctas += (2ll * batch * n_kv_heads + 31) / 32;
    if (ctas > 0x7fffffffll) return MFAR_ERR_LIMIT;
    rope_append_kernel<<<static_cast<unsigned>(ctas), 64, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(qkv), inv_freq, pos_dev, pos, slot_dev, slot, batch, n_q_heads, n_kv_heads,
        static_cast<__half*>(q_out), static_cast<__half*>(k_window), static_cast<__half*>(v_window), win_head_stride,
        win_token_stride, window_capacity, dev_status, prune_rank, prune_back);
    return launch_status();
}

extern "C" int mfar_silu_mul_f16(const void* gate_up, void* out, int64_t rows, int width, void* stream) {
    if (rows < 0 || width <= 0 || (width % 2) != 0) return MFAR_ERR_ARG;
    if (rows == 0) return MFAR_OK;
    if (!gate_up || !out) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(gate_up) & 3) || (reinterpret_cast<uintptr_t>(out) & 3)) return MFAR_ERR_ALIGN;
    const int64_t n2 = rows * (width / 2);
    int64_t blocks = (n2 + 255) / 256;
    const int64_t sms = device_sm_count();
    if (blocks > sms * 8) blocks = sms * 8;
    silu_mul_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(gate_up), static_cast<__half*>(out), rows, width);
    return launch_status();
}
