// Single-product kernels over the quantised bitmap cache (2- or 4-bit codes, per-tile or per-32-nonzero
// scale / zero-point) behind the reference-shaped ops, and the entry points of the quantised cache.  The fused
// attention over this cache is the QBITS instantiation of decode_attn.cu.
//
// Same work split as the fp16 single-product kernels (decode.cu): a CTA of 4 warps walks 64-token
// blocks of one kv head for all G query heads; a lane owns one byte of a tile's bitmap.
// Differences:
//   * staging: every thread copies the metadata of "its" K tile and V tile (bitmap, offset,
//     scale, zero) through registers and the tile's code words with 4-byte cp.async into a
//     fixed slot of a double-buffered shared-memory block, one block ahead of the compute;
//   * a lane extracts a 32-bit window of codes that starts at its first rank with one funnel
//     shift; every set bit consumes `bits` bits of the window;
//   * value = (code - zero) * scale in fp32 (the reference's mode-0 arithmetic,
//     kernel_quant/csrc/SpMM_Kernel_Quant.cuh:235-240, without its re-rounding of the product to
//     fp16), with the scale folded into the per-tile coefficients; fp32 accumulation.
#include "decode_common.cuh"


namespace mfar {

constexpr int kQWarps = 4;
constexpr int kQThreads = kQWarps * 32;
constexpr int kQPlanes = kQWarps * 2;   // (warp, pair of lane groups): two lane groups are folded by a shuffle first
static_assert(kQPlanes * 64 >= kQWarps * kD, "the epilogue reuses the score planes as [warp][G][128] floats");

struct QDecodeParams {
    QSparse k, v;
    const __half* q;
    int64_t q_stride;
    int nblk, nsplit, bps, nrec;
    int group32;
    int kv_share;          // grid rows (groups of query heads) that share one kv head; 0 is read as 1
    float scale_log2;
    float* ws;
    __half* s_out;
    int64_t s_stride;
    const __half* p_in;
    int64_t p_stride;
    unsigned* dev_status;
};

__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// One tile step over quantised codes.  The dequantised value (code - zero) * scale is never
// materialised: per tile the lane folds the scale into the G coefficients (sc[g] = scale * coef[g])
// and per set bit computes d = code - zero exactly (the code is turned into a float by or-ing it into
// the mantissa of 2^23) and accumulates d * sc[g] in fp32.
template <int G, int BITS, bool GROUP32>
__device__ __forceinline__ void tile_step_q(unsigned hi, unsigned lo, const unsigned* words, const unsigned* sz,
                                            unsigned sel, unsigned mh, unsigned ml,
                                            const float (&coef)[G], float (&acc)[8][G]) {
    constexpr unsigned MASK = (1u << BITS) - 1u;
    const unsigned byte = __byte_perm(lo, hi, sel);
    int rank = __popc(hi & mh) + __popc(lo & ml);
    const unsigned bitoff = static_cast<unsigned>(rank) * BITS;
    unsigned window = __funnelshift_r(words[bitoff >> 5], words[(bitoff >> 5) + 1], bitoff & 31u);
    const unsigned sz0 = sz[0];
    const float s0 = __half2float(__ushort_as_half(static_cast<unsigned short>(sz0 & 0xffffu)));
    const float zz0 = 8388608.f + __half2float(__ushort_as_half(static_cast<unsigned short>(sz0 >> 16)));
    if (!GROUP32) {
        float sc[G];
#pragma unroll
        for (int g = 0; g < G; ++g) sc[g] = s0 * coef[g];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (byte & (0x80u >> i)) {
                const float d = __uint_as_float(0x4b000000u | (window & MASK)) - zz0;
                window >>= BITS;
#pragma unroll
                for (int g = 0; g < G; ++g) acc[i][g] = fmaf(d, sc[g], acc[i][g]);
            }
        }
    } else {
        const unsigned sz1 = sz[1];
        const float s1 = __half2float(__ushort_as_half(static_cast<unsigned short>(sz1 & 0xffffu)));
        const float zz1 = 8388608.f + __half2float(__ushort_as_half(static_cast<unsigned short>(sz1 >> 16)));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (byte & (0x80u >> i)) {
                const bool second = rank >= 32;      // nonzeros 32.. of the tile use the second scale / zero
                ++rank;
                const float d = (__uint_as_float(0x4b000000u | (window & MASK)) - (second ? zz1 : zz0)) * (second ? s1 : s0);
                window >>= BITS;
#pragma unroll
                for (int g = 0; g < G; ++g) acc[i][g] = fmaf(d, coef[g], acc[i][g]);
            }
        }
    }
}

template <int G, int MODE, int BITS>
struct QLayout {
    size_t kbuf, vbuf, qh, spart, ps, alpha, total;
    __host__ __device__ QLayout() {
        size_t o = 0;
        kbuf = o; o += (MODE != MODE_VALUE) ? 2 * sizeof(QBuf<BITS>) : 0;
        vbuf = o; o += (MODE != MODE_KEY) ? 2 * sizeof(QBuf<BITS>) : 0;
        qh = o;    o += kD * G * 4;
        spart = o; o += static_cast<size_t>(kQPlanes) * G * 64 * 4;
        ps = o;    o += 64 * G * 4 + 64;
        alpha = o; o += 64;
        total = o;
    }
};

template <int G, int MODE, int BITS, bool GROUP32>
__global__ void __launch_bounds__(kQThreads, 4) decode_quant_kernel(QDecodeParams p) {
    constexpr int CAP = 32 / BITS;
    constexpr int WPT = QBuf<BITS>::WPT;
    extern __shared__ __align__(128) unsigned char smem[];
    const QLayout<G, MODE, BITS> lay;
    QBuf<BITS>* kbuf = reinterpret_cast<QBuf<BITS>*>(smem + lay.kbuf);
    QBuf<BITS>* vbuf = reinterpret_cast<QBuf<BITS>*>(smem + lay.vbuf);
    float* qh = reinterpret_cast<float*>(smem + lay.qh);                    // [128][G]
    float* spart = reinterpret_cast<float*>(smem + lay.spart);              // [plane][G][64]
    float* ps = reinterpret_cast<float*>(smem + lay.ps);                    // [64][G]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // hq numbers the (kv head, group of G query heads) pairs; with kv_share > 1 several of them read the same kv head
    const int hq = blockIdx.y, split = blockIdx.x;
    const int h = hq / (p.kv_share > 0 ? p.kv_share : 1);
    const int gi = lane >> 3, kb = lane & 7;
    unsigned sel, mh, ml;
    lane_byte_constants(kb, sel, mh, ml);
    const int blk0 = split * p.bps;
    const int nb = max(0, min(p.bps, p.nblk - blk0));
    const int ngrp = GROUP32 ? 2 : 1;

    if (MODE != MODE_VALUE) {
        for (int i = tid; i < kD * G; i += kQThreads) {
            const int c = i / G, g = i % G;
            qh[i] = __half2float(p.q[(static_cast<int64_t>(hq) * G + g) * p.q_stride + c]);
        }
    }

    // ---- staging: thread t owns K tile t and V tile t of a block
    struct Meta { uint2 bm; int off; unsigned sz[2]; };
    Meta mk{}, mv{};
    auto load_meta = [&](const QSparse& s, int i, Meta& m) {
        const int64_t t = static_cast<int64_t>(blk0 + i) * kTilesPerBlock + tid;
        const unsigned long long b = s.bmp[h * s.bmp_hs + t];
        m.bm = make_uint2(static_cast<unsigned>(b), static_cast<unsigned>(b >> 32));
        const int64_t mi = h * s.meta_hs + t;
        m.off = s.tile_off[mi];
        for (int g = 0; g < ngrp; ++g)
            m.sz[g] = static_cast<unsigned>(__half_as_ushort(s.scales[mi * ngrp + g])) |
                      (static_cast<unsigned>(__half_as_ushort(s.zeros[mi * ngrp + g])) << 16);
    };
    auto stage = [&](const QSparse& s, const Meta& m, QBuf<BITS>& b) {
        b.bm[tid] = m.bm;
        b.sz[2 * tid] = m.sz[0];
        b.sz[2 * tid + 1] = m.sz[1];
        const int n = (__popc(m.bm.x) + __popc(m.bm.y) + CAP - 1) / CAP;
        if (m.off < 0 || static_cast<long long>(m.off) + n > s.packed_words) {
            if (n > 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_BADMETA);
            b.bm[tid] = make_uint2(0u, 0u);     // the tile contributes nothing
            return;
        }
        const unsigned* src = s.packed + m.off;
        for (int j = 0; j < n; ++j) cp_async4(&b.words[tid * WPT + j], src + j);
    };
    if (nb > 0) {
        if (MODE != MODE_VALUE) { load_meta(p.k, 0, mk); stage(p.k, mk, kbuf[0]); }
        if (MODE != MODE_KEY) { load_meta(p.v, 0, mv); stage(p.v, mv, vbuf[0]); }
        cp_async_commit();
        if (nb > 1) {
            if (MODE != MODE_VALUE) load_meta(p.k, 1, mk);
            if (MODE != MODE_KEY) load_meta(p.v, 1, mv);
        }
    }

    float acc_o[8][G];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int g = 0; g < G; ++g) acc_o[i][g] = 0.f;
    constexpr int kHeadsPerWarp = (G + kQWarps - 1) / kQWarps;

    for (int i = 0; i < nb; ++i) {
        cp_async_wait_all();
        __syncthreads();   // block i has landed for everybody; everybody is done with block i-1
        if (i + 1 < nb) {
            if (MODE != MODE_VALUE) stage(p.k, mk, kbuf[(i + 1) & 1]);
            if (MODE != MODE_KEY) stage(p.v, mv, vbuf[(i + 1) & 1]);
            cp_async_commit();
            if (i + 2 < nb) {
                if (MODE != MODE_VALUE) load_meta(p.k, i + 2, mk);
                if (MODE != MODE_KEY) load_meta(p.v, i + 2, mv);
            }
        }
        const QBuf<BITS>& kbf = kbuf[i & 1];
        const QBuf<BITS>& vbf = vbuf[i & 1];

        // ------------------------------------------------------------ K phase
        if (MODE != MODE_VALUE) {
            float acc_s[8][G];
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int g = 0; g < G; ++g) acc_s[t][g] = 0.f;
#pragma unroll 8
            for (int s = 0; s < 32 / 4; ++s) {
                const int c = warp * 32 + s * 4 + gi;
                const uint2 bm = kbf.bm[c];
                float coef[G];
                load_coef<G>(qh + c * G, coef);
                tile_step_q<G, BITS, GROUP32>(bm.y, bm.x, kbf.words + c * WPT, kbf.sz + 2 * c, sel, mh, ml, coef, acc_s);
            }
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int g = 0; g < G; ++g) acc_s[t][g] += __shfl_xor_sync(kFull, acc_s[t][g], 16);
            if (gi < 2) {
                float* dst = spart + (static_cast<size_t>(warp * 2 + gi) * G) * 64 + kb * 8;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    *reinterpret_cast<float4*>(dst + g * 64) = make_float4(acc_s[0][g], acc_s[1][g], acc_s[2][g], acc_s[3][g]);
                    *reinterpret_cast<float4*>(dst + g * 64 + 4) = make_float4(acc_s[4][g], acc_s[5][g], acc_s[6][g], acc_s[7][g]);
                }
            }
            __syncthreads();
        }

        // ------------------------------------------------------------ scores -> probabilities
        if (MODE == MODE_VALUE) {
            for (int g = warp; g < G; g += kQWarps) {
                const unsigned pv = *reinterpret_cast<const unsigned*>(
                    p.p_in + (static_cast<int64_t>(hq) * G + g) * p.p_stride + static_cast<int64_t>(blk0 + i) * 64 + 2 * lane);
                ps[(2 * lane) * G + g] = __half2float(__ushort_as_half(static_cast<unsigned short>(pv & 0xffffu)));
                ps[(2 * lane + 1) * G + g] = __half2float(__ushort_as_half(static_cast<unsigned short>(pv >> 16)));
            }
        } else {
#pragma unroll
            for (int j = 0; j < kHeadsPerWarp; ++j) {
                const int g = warp + j * kQWarps;
                if (g < G) {
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int pl = 0; pl < kQPlanes; ++pl) {
                        const float2 t = *reinterpret_cast<const float2*>(spart + (static_cast<size_t>(pl) * G + g) * 64 + 2 * lane);
                        s0 += t.x;
                        s1 += t.y;
                    }
                    // MODE_KEY (the only mode that gets here): the scores leave as they are
                    *reinterpret_cast<__half2*>(p.s_out + (static_cast<int64_t>(hq) * G + g) * p.s_stride +
                                                static_cast<int64_t>(blk0 + i) * 64 + 2 * lane) = __floats2half2_rn(s0, s1);
                }
            }
        }
        if (MODE == MODE_KEY) continue;
        __syncthreads();

        // ------------------------------------------------------------ V phase
        const int half_id = gi & 1, par = gi >> 1;
#pragma unroll 8
        for (int s = 0; s < 16 / 2; ++s) {
            const int t = warp * 16 + s * 2 + par;
            const int tile = half_id * 64 + t;
            const uint2 bm = vbf.bm[tile];
            float coef[G];
            load_coef<G>(ps + t * G, coef);
            tile_step_q<G, BITS, GROUP32>(bm.y, bm.x, vbf.words + tile * WPT, vbf.sz + 2 * tile, sel, mh, ml, coef, acc_o);
        }
    }
    if (MODE == MODE_KEY) return;

    __syncthreads();
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int g = 0; g < G; ++g) acc_o[t][g] += __shfl_xor_sync(kFull, acc_o[t][g], 16);
    float* red = spart;
    if (lane < 16) {
        const int ch = (gi & 1) * 64 + kb * 8;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float* d = red + (static_cast<size_t>(warp) * G + g) * kD + ch;
            *reinterpret_cast<float4*>(d) = make_float4(acc_o[0][g], acc_o[1][g], acc_o[2][g], acc_o[3][g]);
            *reinterpret_cast<float4*>(d + 4) = make_float4(acc_o[4][g], acc_o[5][g], acc_o[6][g], acc_o[7][g]);
        }
    }
    __syncthreads();
    float* rec = p.ws + ((static_cast<int64_t>(hq) * p.nrec + split) * G) * kPartialStride;
    for (int idx = tid; idx < G * kD; idx += kQThreads) {
        const int g = idx / kD, c = idx % kD;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kQWarps; ++w) s += red[(static_cast<size_t>(w) * G + g) * kD + c];
        rec[g * kPartialStride + c] = s;
    }
}

template <int G, int MODE, int BITS, bool GROUP32>
static int launch_q(const QDecodeParams& p, int n_kv_heads, cudaStream_t s) {
    const QLayout<G, MODE, BITS> lay;
    static bool configured[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MFAR_ERR_LAUNCH;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(decode_quant_kernel<G, MODE, BITS, GROUP32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(lay.total)) != cudaSuccess)
            return MFAR_ERR_LAUNCH;
        configured[dev] = true;
    }
    decode_quant_kernel<G, MODE, BITS, GROUP32><<<dim3(p.nsplit, n_kv_heads), kQThreads, lay.total, s>>>(p);
    return launch_status();
}

template <int MODE>
static int dispatch_q(const QDecodeParams& p, int G, int bits, int n_kv_heads, cudaStream_t s) {
#define MFAR_QCASE(GG)                                                                      \
    case GG:                                                                                \
        if (bits == 2) return p.group32 ? launch_q<GG, MODE, 2, true>(p, n_kv_heads, s)     \
                                        : launch_q<GG, MODE, 2, false>(p, n_kv_heads, s);   \
        return p.group32 ? launch_q<GG, MODE, 4, true>(p, n_kv_heads, s)                    \
                         : launch_q<GG, MODE, 4, false>(p, n_kv_heads, s);
    switch (G) {
        MFAR_QCASE(1)
        MFAR_QCASE(2)
        MFAR_QCASE(4)
        case 8: {
            // 64 accumulators per phase spill; two CTAs of 4 query heads each share the kv head instead
            // (records then lie as [kv head * 2 + half][record][4]: combine with G = 4)
            QDecodeParams p2 = p;
            p2.kv_share = 2;
            return dispatch_q<MODE>(p2, 4, bits, 2 * n_kv_heads, s);
        }
        default: return MFAR_ERR_ARG;
    }
#undef MFAR_QCASE
}

static int check_q(const void* bmp, const void* off, const void* sc, const void* ze, const void* packed, int bits, int qgroup) {
    if (!bmp || !off || !sc || !ze || !packed) return MFAR_ERR_ARG;
    if ((bits != 2 && bits != 4) || (qgroup != 32 && qgroup != 64)) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(bmp) & 7) || (reinterpret_cast<uintptr_t>(off) & 3) ||
        (reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(sc) & 1) || (reinterpret_cast<uintptr_t>(ze) & 1))
        return MFAR_ERR_ALIGN;
    return MFAR_OK;
}

static void q_split(int n_kv_heads, int nblk, int hint, int* ns, int* bps) {
    const int max_n = (nblk + 1) / 2;   // what callers size their workspace for
    int n = hint > 0 ? hint : model_split_count(n_kv_heads, nblk, 1, max_n < 128 ? max_n : 128, device_sm_count());
    if (n > nblk) n = nblk;
    if (n < 1) n = 1;
    *bps = (nblk + n - 1) / n;
    *ns = (nblk + *bps - 1) / *bps;
}

}  // namespace mfar

using namespace mfar;

extern "C" int mfar_key_scores_quant(const void* q, int64_t q_stride, int n_kv_heads, int group,
                                     const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* tile_offsets,
                                     const void* scales, const void* zeros, int64_t meta_head_stride,
                                     const int32_t* packed, int64_t packed_words, int n_tokens, int bits, int qgroup,
                                     void* scores, int64_t scores_stride, uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens < 0 || (n_tokens % 64) || packed_words < 0) return MFAR_ERR_ARG;
    if (n_tokens == 0) return MFAR_OK;
    if (!q || !scores) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(scores) & 3) || (scores_stride & 1)) return MFAR_ERR_ALIGN;
    int r = check_q(bitmaps, tile_offsets, scales, zeros, packed, bits, qgroup);
    if (r) return r;
    QDecodeParams p{};
    p.k = QSparse{reinterpret_cast<const unsigned long long*>(bitmaps), tile_offsets, static_cast<const __half*>(scales),
                  static_cast<const __half*>(zeros), reinterpret_cast<const unsigned*>(packed), bmp_head_stride,
                  meta_head_stride, packed_words};
    p.q = static_cast<const __half*>(q);
    p.q_stride = q_stride;
    p.nblk = n_tokens / 64;
    q_split(n_kv_heads, p.nblk, 0, &p.nsplit, &p.bps);
    p.group32 = qgroup == 32;
    p.s_out = static_cast<__half*>(scores);
    p.s_stride = scores_stride;
    p.dev_status = dev_status;
    return dispatch_q<MODE_KEY>(p, group, bits, n_kv_heads, static_cast<cudaStream_t>(stream));
}

extern "C" int mfar_value_output_quant(const void* probs, int64_t probs_stride, int n_kv_heads, int group,
                                       const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* tile_offsets,
                                       const void* scales, const void* zeros, int64_t meta_head_stride,
                                       const int32_t* packed, int64_t packed_words, int n_tokens, int bits, int qgroup,
                                       void* out, int64_t out_stride, void* workspace, size_t workspace_bytes,
                                       int nsplit, uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens <= 0 || (n_tokens % 64) || packed_words < 0) return MFAR_ERR_ARG;
    if (!probs || !out || !workspace) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(probs) & 3) || (probs_stride & 1)) return MFAR_ERR_ALIGN;
    int r = check_q(bitmaps, tile_offsets, scales, zeros, packed, bits, qgroup);
    if (r) return r;
    QDecodeParams p{};
    p.v = QSparse{reinterpret_cast<const unsigned long long*>(bitmaps), tile_offsets, static_cast<const __half*>(scales),
                  static_cast<const __half*>(zeros), reinterpret_cast<const unsigned*>(packed), bmp_head_stride,
                  meta_head_stride, packed_words};
    p.nblk = n_tokens / 64;
    q_split(n_kv_heads, p.nblk, nsplit, &p.nsplit, &p.bps);
    p.nrec = p.nsplit;
    const size_t need = counters_bytes(n_kv_heads) + static_cast<size_t>(n_kv_heads) * p.nrec * group * kPartialStride * sizeof(float);
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return MFAR_ERR_WORKSPACE;
    p.group32 = qgroup == 32;
    p.p_in = static_cast<const __half*>(probs);
    p.p_stride = probs_stride;
    p.ws = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + counters_bytes(n_kv_heads));
    p.dev_status = dev_status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    r = dispatch_q<MODE_VALUE>(p, group, bits, n_kv_heads, s);
    if (r) return r;
    return launch_combine(p.ws, p.nrec, group == 8 ? 4 : group, 0, out, out_stride, n_kv_heads * group, s);
}

extern "C" int mfar_decode_attention_quant(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, const int32_t* k_tile_offsets, const void* k_scales, const void* k_zeros,
    const int32_t* k_packed, int64_t k_packed_words,
    const int64_t* v_bitmaps, const int32_t* v_tile_offsets, const void* v_scales, const void* v_zeros,
    const int32_t* v_packed, int64_t v_packed_words,
    int64_t bmp_head_stride, int64_t meta_head_stride, int n_tokens, const int32_t* n_tokens_dev, int bits, int qgroup,
    const void* k_window, const void* v_window, int64_t win_head_stride, int64_t win_token_stride, int window,
    const int32_t* window_len_dev, float softmax_scale, void* out, int64_t out_stride, void* workspace,
    size_t workspace_bytes, int nsplit, uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens < 0 || (n_tokens % 64) || window < 0) return MFAR_ERR_ARG;
    if (n_tokens == 0 && window == 0) return MFAR_ERR_ARG;
    if (group != 1 && group != 2 && group != 4 && group != 8) return MFAR_ERR_ARG;
    if (!q || !out || !workspace) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(q) & 3) || (q_stride & 1)) return MFAR_ERR_ALIGN;
    if (window > 0 && (!k_window || !v_window)) return MFAR_ERR_ARG;
    if (window > 0 && ((reinterpret_cast<uintptr_t>(k_window) & 15) || (reinterpret_cast<uintptr_t>(v_window) & 15) ||
                       (win_head_stride & 7) || (win_token_stride & 7)))
        return MFAR_ERR_ALIGN;
    if ((bits != 2 && bits != 4) || (qgroup != 32 && qgroup != 64)) return MFAR_ERR_ARG;
    DecodeParams p{};
    int r;
    if (n_tokens > 0) {
        r = check_q(k_bitmaps, k_tile_offsets, k_scales, k_zeros, k_packed, bits, qgroup);
        if (r) return r;
        r = check_q(v_bitmaps, v_tile_offsets, v_scales, v_zeros, v_packed, bits, qgroup);
        if (r) return r;
        p.nblk = n_tokens / 64;
        q_split(n_kv_heads, p.nblk, nsplit, &p.nsplit, &p.bps);
    }
    p.nrec = p.nsplit + (window > 0 ? 1 : 0);
    const size_t need = counters_bytes(n_kv_heads) + static_cast<size_t>(n_kv_heads) * p.nrec * group * kPartialStride * sizeof(float);
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return MFAR_ERR_WORKSPACE;
    p.kq = QSparse{reinterpret_cast<const unsigned long long*>(k_bitmaps), k_tile_offsets,
                   static_cast<const __half*>(k_scales), static_cast<const __half*>(k_zeros),
                   reinterpret_cast<const unsigned*>(k_packed), bmp_head_stride, meta_head_stride, k_packed_words};
    p.vq = QSparse{reinterpret_cast<const unsigned long long*>(v_bitmaps), v_tile_offsets,
                   static_cast<const __half*>(v_scales), static_cast<const __half*>(v_zeros),
                   reinterpret_cast<const unsigned*>(v_packed), bmp_head_stride, meta_head_stride, v_packed_words};
    p.q = static_cast<const __half*>(q);
    p.q_stride = q_stride;
    p.kwin = static_cast<const __half*>(k_window);
    p.vwin = static_cast<const __half*>(v_window);
    p.win_hs = win_head_stride;
    p.win_ts = win_token_stride;
    p.W = window;
    p.W_dev = window_len_dev;
    p.L_dev = n_tokens_dev;
    p.cap = 8;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.counters = n_kv_heads <= kMaxCountedHeads ? static_cast<unsigned*>(workspace) : nullptr;
    p.ws = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + counters_bytes(n_kv_heads));
    p.out = static_cast<__half*>(out);
    p.out_stride = out_stride;
    p.dev_status = dev_status;
    p.rec_group = group;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    r = launch_decode_attn_quant(p, group, bits, qgroup == 32, n_kv_heads, p.nrec, s);
    if (r || p.counters) return r;
    return launch_combine(p.ws, p.nrec, group, 1, out, out_stride, n_kv_heads * group, s);
}
