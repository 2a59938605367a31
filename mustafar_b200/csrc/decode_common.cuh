// Building blocks shared by the fp16 and the quantised decode kernels:
// mbarrier / bulk-copy wrappers (1-D cp.async.bulk, no multicast), the position-centric
// tile step, the split-KV partial record and the launch parameters.
#pragma once

#include "common.cuh"

namespace mfar {

// ---------------------------------------------------------------- mbarrier + TMA 1-D bulk copy
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out (caller records MFAR_DEV_TIMEOUT and leaves).
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > kWaitLimitNs) return false;
    }
}
// global -> this CTA's shared memory; src/dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// ---------------------------------------------------------------- small math helpers
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float warp_max_f32(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, d));
    return v;
}
__device__ __forceinline__ float warp_sum_f32(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(kFull, v, d);
    return v;
}

// One tile step for one lane.  `hi:lo` is the tile's 64-bit bitmap (bit 63-i = element i),
// `vals` its packed values in shared memory.  The lane owns byte `kb` of the bitmap, i.e.
// positions 8*kb .. 8*kb+7: sel / mh / ml are the lane constants that extract that byte and
// mask the bits in front of it.  The rank of the lane's first position is the popcount of
// the bits before its byte; every set bit then consumes the next packed half and is
// multiply-accumulated in fp32 into acc[i][g] with the per-tile coefficients coef[g]
// (K phase: the query channel; V phase: the probability of the token).  The compiler turns
// the `if` into predicated instructions (no branch, no zero fill).
__device__ __forceinline__ void lane_byte_constants(int kb, unsigned& sel, unsigned& mh, unsigned& ml) {
    sel = 7u - kb;
    mh = kb == 0 ? 0u : (kb >= 4 ? 0xffffffffu : (0xffffffffu << (32 - 8 * kb)));
    ml = kb <= 4 ? 0u : (0xffffffffu << (64 - 8 * kb));
}

__device__ __forceinline__ float fma_h(float acc, unsigned short a, unsigned short b) {
    asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(a), "h"(b));
    return acc;
}

// The packed half and the fp16 coefficient go straight into one mixed-precision FMA (fp16 x fp16 + fp32, full rate
// on sm_100).  Two read pointers (positions 0-3 and 4-7) keep the dependent chain of pointer bumps short.
template <int G>
__device__ __forceinline__ void tile_step(unsigned hi, unsigned lo, const unsigned short* vals, unsigned sel,
                                          unsigned mh, unsigned ml, const unsigned short (&coef)[G], float (&acc)[8][G]) {
    const unsigned byte = __byte_perm(lo, hi, sel);
    const unsigned short* pv[2];
    pv[0] = vals + (__popc(hi & mh) + __popc(lo & ml));
    pv[1] = pv[0] + __popc(byte & 0xf0u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (byte & (0x80u >> i)) {
            const unsigned short*& p = pv[i / 4];
            const unsigned short v = *p;
            ++p;
#pragma unroll
            for (int g = 0; g < G; ++g) acc[i][g] = fma_h(acc[i][g], v, coef[g]);
        }
    }
}

template <int G>
__device__ __forceinline__ void load_coef(const float* p, float (&c)[G]) {
    if constexpr (G == 1) {
        c[0] = p[0];
    } else if constexpr (G == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        c[0] = t.x; c[1] = t.y;
    } else {
#pragma unroll
        for (int g = 0; g < G; g += 4) {
            const float4 t = *reinterpret_cast<const float4*>(p + g);
            c[g] = t.x; c[g + 1] = t.y; c[g + 2] = t.z; c[g + 3] = t.w;
        }
    }
}

template <int G>
__device__ __forceinline__ void load_coef(const unsigned short* p, unsigned short (&c)[G]) {
    if constexpr (G == 1) {
        c[0] = p[0];
    } else if constexpr (G == 2) {
        const unsigned t = *reinterpret_cast<const unsigned*>(p);
        c[0] = t & 0xffffu; c[1] = t >> 16;
    } else {
#pragma unroll
        for (int g = 0; g < G; g += 4) {
            const uint2 t = *reinterpret_cast<const uint2*>(p + g);
            c[g] = t.x & 0xffffu; c[g + 1] = t.x >> 16; c[g + 2] = t.y & 0xffffu; c[g + 3] = t.y >> 16;
        }
    }
}

__device__ __forceinline__ void store_coef(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_coef(unsigned short* p, float v) { *p = __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ float coef_value(float v) { return v; }
// the probability that enters P.V is the fp16-rounded one; the running sum must use the same value
__device__ __forceinline__ float round_like(const unsigned short*, float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float round_like(const float*, float v) { return v; }

__device__ __forceinline__ float coef_to_float(float v) { return v; }
__device__ __forceinline__ float coef_to_float(unsigned short v) { return __half2float(__ushort_as_half(v)); }

// Split-KV partial of one (kv head, split, q head of the group): 128 un-normalised
// output channels, then the running max (log2 domain) and the running sum.
constexpr int kPartialStride = kD + 4;  // floats; keeps records 16-byte aligned
constexpr int kPartM = kD;
constexpr int kPartL = kD + 1;

enum { MODE_KEY = 1, MODE_VALUE = 2 };
constexpr int kSlackHalves = 64;  // a decode never reads further than this past a stage's values
constexpr int kMaxBlocksPerSplit = 256;

struct Sparse {
    const unsigned long long* bmp;
    const int* acc;
    const __half* nz;
    const int* nz_off;
    int64_t bmp_hs, acc_hs, nz_hs;
    int64_t nz_extent;   // halves addressable from nz (0 = unknown: the extent check is skipped)
};

// one tensor of the quantised cache (mfar_compress_quant)
struct QSparse {
    const unsigned long long* bmp;
    const int* tile_off;
    const __half* scales;
    const __half* zeros;
    const unsigned* packed;
    int64_t bmp_hs, meta_hs;
    long long packed_words;
};

template <int BITS_>
struct QBuf {   // one staged tensor of one 64-token block of the quantised cache
    static constexpr int BITS = BITS_;
    static constexpr int WPT = 64 * BITS_ / 32;  // words per tile slot
    uint2 bm[128];
    unsigned sz[128 * 2];                        // (scale | zero << 16) per group
    unsigned words[128 * WPT + 4];
};

struct DecodeParams {
    Sparse k, v;
    QSparse kq, vq;        // fused attention over the quantised cache (k, v unused then)
    const __half* q;       // [Bq][q_stride]
    int64_t q_stride;
    const __half* kwin;    // dense window [Bh][W][128]
    const __half* vwin;
    int64_t win_hs, win_ts;
    int W;
    const int* W_dev;      // optional: window length in device memory (then W is its upper bound)
    const int* L_dev;      // optional: compressed tokens in device memory (then nblk is their upper bound, in blocks)
    int nblk, nsplit, bps; // compressed blocks, splits over them, blocks per split
    int cap;               // halves of packed values a stage can hold per tensor
    float scale_log2;      // softmax scale * log2(e)
    float* ws;             // split partials
    int nrec;              // partial records per kv head in ws
    int rec_group;         // query heads per record set: G, or 4 when 8 heads are laid out as two sets of 4
    __half* s_out;         // MODE_KEY  : [Bq][s_stride]
    int64_t s_stride;
    const __half* p_in;    // MODE_VALUE: [Bq][p_stride]
    int64_t p_stride;
    unsigned* dev_status;
    int split_offset;      // added to blockIdx.x (lets a launch cover only the window record)
    int kv_share;          // single-product kernels: grid rows (sets of query heads) sharing one kv head; 0 reads as 1
    // fused attention only: the CTA that finishes a kv head last merges its records into out
    unsigned* counters;    // one per kv head, zero between launches; NULL = no merge (a combine launch follows)
    __half* out;
    int64_t out_stride;
};

// The first kCounterBytes of every decode workspace hold one arrival counter per kv head (fused attention); the
// split records of every entry point start behind them, whatever the head count, so that calls of different shapes
// can share a workspace without touching each other's counters.
constexpr size_t kCounterBytes = 64 * 1024;
constexpr int kMaxCountedHeads = static_cast<int>(kCounterBytes / 4);
inline size_t counters_bytes(int) { return kCounterBytes; }

// Checks one 64-token block's packed range before it is copied: block start `blk` and end `nxt` in uint32 units
// (entries of accum), stage capacity `capb` in bytes, start of the head inside nz and the extent of nz in halves.
// A bulk copy needs a 16-byte aligned source and a size that is a multiple of 16 bytes.
__device__ __forceinline__ bool block_range_bad(int blk, int nxt, unsigned capb, int64_t head_start_halves,
                                                int64_t nz_extent) {
    const long long d = (static_cast<long long>(nxt) - blk) * 4;
    bool bad = d < 0 || d > capb || blk < 0 || (blk & 3) || (d & 15);
    if (nz_extent > 0) bad |= head_start_halves + 2ll * nxt > nz_extent;
    return bad;
}

// fused decode attention (decode_attn.cu): grid (grid_x, n_kv_heads); G in {1, 2, 4, 8}
int launch_decode_attn(const DecodeParams& p, int G, int n_kv_heads, int grid_x, cudaStream_t s);
// the same over the quantised cache p.kq / p.vq: bits in {2, 4}, group32 = a second scale / zero-point from nonzero 32 on
int launch_decode_attn_quant(const DecodeParams& p, int G, int bits, bool group32, int n_kv_heads, int grid_x,
                             cudaStream_t s);
// merge of the split-KV records (normalise = 1) or plain sum (normalise = 0), one CTA per q head
int launch_combine(const float* ws, int nrec, int G, int normalise, void* out, int64_t out_stride, int n_q_heads,
                   cudaStream_t s);
// Split count of the 64-token-block decode kernels.  The grid is n_kv_heads * ns CTAs of bps = ceil(nblk / ns) blocks.
// The cost of a candidate follows a model fitted to a measured sweep of ns over batch 1..64 and
// 4k..32k tokens on a B200 (all times in units of one block on an otherwise idle SM, ~2 us):
//   * a CTA costs w = bps + 1.1 (prologue, partial record);
//   * x = CTAs / SMs is the load per SM; an SM's throughput with o = min(x, 4) resident CTAs is
//     rate(o) = 1 / 2 / 2.76 / 2.13 at o = 1 / 2 / 3 / 4, linear in between (the dip at 4 is the fit's
//     way of saying that a grid which fits in one not-quite-full wave beats one that needs two);
//   * the last, partly filled wave costs another 0.8 w once the SMs hold more than one CTA;
//   * merging the records adds 0.035 per record.
// The pick stays within 2 % of the best swept ns on every measured shape.
inline int model_split_count(int n_kv_heads, int nblk, int min_ns, int max_ns, int n_sm) {
    if (max_ns > nblk) max_ns = nblk;
    if (min_ns < 1) min_ns = 1;
    if (n_sm < 1) n_sm = 1;
    int ns = min_ns;
    double best = -1.0;
    for (int cand = min_ns; cand <= max_ns; ++cand) {
        const int bps = (nblk + cand - 1) / cand;
        const int real = (nblk + bps - 1) / bps;
        const double x = static_cast<double>(n_kv_heads) * real / n_sm;
        const double w = bps + 1.1;
        double cost = w;
        if (x > 1.0) {
            const double o = x < 4.0 ? x : 4.0;
            const double rate = o < 2.0 ? o : (o < 3.0 ? 2.0 + 0.76 * (o - 2.0) : 2.76 - 0.63 * (o - 3.0));
            cost = x * w / rate + 0.8 * w * (x - 1.0 < 1.0 ? x - 1.0 : 1.0);
        }
        cost += 0.035 * real;
        if (best < 0 || cost < best) {
            best = cost;
            ns = real;
        }
    }
    return ns;
}

}  // namespace mfar
