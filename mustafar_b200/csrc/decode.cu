// Decode entry points over the bitmap + packed-fp16 cache, and the two single-product kernels behind the
// reference-shaped ops:
//   KEY    S = K~ q       (what mustafar_key_formulation returns in row 0)
//   VALUE  O = V~^T p     (what mustafar_value_formulation returns in row 0)
// The fused attention kernel lives in decode_attn.cu.
//
// spmv_kernel: a CTA (4 warps) walks a range of 64-token blocks of ONE kv head and serves all G query heads that
// share it.  Per block the bitmap array (1 KiB) and the packed-value range travel into a 2-stage shared-memory
// ring by 1-D bulk copies (cp.async.bulk + mbarrier, no multicast), issued by one thread one block ahead.  Tiles
// are decoded straight from the bitmap: a lane owns one BYTE of a tile's bitmap (8 positions), 8 lanes cover a
// tile, a warp does 4 tiles per step; the rank of the lane's first position is the popcount of the bits before its
// byte; every set bit takes the next packed half and is multiply-accumulated in fp32 for all G heads.
// KEY: lane owns 8 tokens, loops over its warp's 32 channels.  VALUE: lane owns 8 channels, loops over its warp's
// 16 tokens; split partials are summed by combine_kernel.
#include "decode_common.cuh"

namespace mfar {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 2;
// KEY partial planes: (warp, lane group), halved by the shuffle stage that folds two lane groups first
constexpr int kGroupsPerWarp = 2;
constexpr int kPlanes = kWarps * kGroupsPerWarp;

__host__ __device__ inline size_t stage_bytes(int cap) { return 1024 + (static_cast<size_t>(cap) + kSlackHalves) * 2; }

template <int G>
struct SmemLayout {
    size_t stages, bars, qs, spart, ps, off, blk, total;
    __host__ __device__ explicit SmemLayout(int cap) {
        size_t o = 0;
        stages = o; o += kStages * stage_bytes(cap);
        bars = o;   o += 64;
        qs = o;     o += kD * G * 2;
        spart = o;  o += static_cast<size_t>(kPlanes) * G * 64 * 4;   // KEY: score planes; VALUE: [warp][G][128] reduction
        ps = o;     o += 64 * G * 2;
        off = o;    o += 2 * 128 * 4;
        blk = o;    o += (kMaxBlocksPerSplit + 4) * 4;
        total = o;
    }
};
static_assert(kPlanes * 64 >= kWarps * kD, "the VALUE epilogue reuses the score planes as [warp][G][128] floats");

template <int G, int MODE>
__global__ void __launch_bounds__(kThreads, 4) spmv_kernel(DecodeParams p) {
    static_assert(MODE == MODE_KEY || MODE == MODE_VALUE, "single-product kernel");
    extern __shared__ __align__(128) unsigned char smem[];
    const SmemLayout<G> lay(p.cap);
    const Sparse& sp = (MODE == MODE_KEY) ? p.k : p.v;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + lay.bars);
    unsigned short* qs = reinterpret_cast<unsigned short*>(smem + lay.qs);      // [128][G] query, fp16
    float* spart = reinterpret_cast<float*>(smem + lay.spart);
    unsigned short* ps = reinterpret_cast<unsigned short*>(smem + lay.ps);      // [64][G] probabilities, fp16
    unsigned* off = reinterpret_cast<unsigned*>(smem + lay.off);                // [2][128] halves, relative to the block
    int* blk = reinterpret_cast<int*>(smem + lay.blk);                          // block starts (uint32 units) of this split

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // hq numbers the (kv head, set of G query heads) pairs; with kv_share > 1 several of them read the same kv head
    const int hq = blockIdx.y;
    const int h = hq / (p.kv_share > 0 ? p.kv_share : 1);
    const int split = blockIdx.x;
    const int gi = lane >> 3, kb = lane & 7;
    unsigned sel, mh, ml;
    lane_byte_constants(kb, sel, mh, ml);

    const int blk0 = split * p.bps;
    int nb = min(p.bps, p.nblk - blk0);
    if (nb < 0) nb = 0;

    if (MODE == MODE_KEY) {
        for (int i = tid; i < kD * G; i += kThreads) {
            const int c = i / G, g = i % G;
            qs[i] = __half_as_ushort(p.q[(static_cast<int64_t>(hq) * G + g) * p.q_stride + c]);
        }
    }
    const int* acc = sp.acc + h * sp.acc_hs;
    for (int i = tid; i <= nb; i += kThreads) blk[i] = acc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const int64_t head0 = sp.nz_off ? 8ll * sp.nz_off[h] : h * sp.nz_hs;
    const __half* nz = sp.nz + head0;
    const size_t stg = stage_bytes(p.cap);
    const unsigned capb = static_cast<unsigned>(p.cap) * 2u;

    auto issue = [&](int i) {
        unsigned char* st = smem + lay.stages + static_cast<size_t>(i % kStages) * stg;
        unsigned long long* bar = &bars[i % kStages];
        const int64_t tile0 = static_cast<int64_t>(blk0 + i) * kTilesPerBlock;
        unsigned bytes = static_cast<unsigned>(blk[i + 1] - blk[i]) * 4u;
        if (block_range_bad(blk[i], blk[i + 1], capb, head0, sp.nz_extent)) {   // the bitmaps are still copied
            if (p.dev_status) atomicOr(p.dev_status, MFAR_DEV_BADMETA);
            bytes = 0;
        }
        mbar_expect_tx(bar, 1024 + bytes);
        bulk_g2s(st, sp.bmp + h * sp.bmp_hs + tile0, 1024, bar);
        if (bytes) bulk_g2s(st + 1024, nz + 2ll * blk[i], bytes, bar);
    };
    int nxt = 0;
    auto fetch_offsets = [&](int i) { nxt = acc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock + tid]; };
    auto store_offsets = [&](int i) {
        off[(i & 1) * 128 + tid] = min(static_cast<unsigned>(2 * (nxt - blk[i])), static_cast<unsigned>(p.cap));
    };
    if (nb > 0) {
        if (tid == 0)
            for (int i = 0; i < min(nb, kStages - 1); ++i) issue(i);
        fetch_offsets(0);
        store_offsets(0);
    }
    __syncthreads();

    float acc_o[8][G];   // VALUE: channels 64*(gi&1) + 8*kb + i, summed over this lane's tokens
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int g = 0; g < G; ++g) acc_o[i][g] = 0.f;

    bool timed_out = false;
    for (int i = 0; i < nb; ++i) {
        const unsigned char* st = smem + lay.stages + static_cast<size_t>(i % kStages) * stg;
        const uint2* bm_s = reinterpret_cast<const uint2*>(st);
        const unsigned short* val = reinterpret_cast<const unsigned short*>(st + 1024);
        const unsigned* of = off + (i & 1) * 128;

        if (i + 1 < nb) fetch_offsets(i + 1);
        if (!mbar_wait(&bars[i % kStages], (i / kStages) & 1)) timed_out = true;
        if (__syncthreads_or(timed_out)) { timed_out = true; break; }   // also publishes the stage hand-off below
        if (tid == 0 && i + kStages - 1 < nb) issue(i + kStages - 1);

        if (MODE == MODE_KEY) {
            float acc_s[8][G];
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int g = 0; g < G; ++g) acc_s[t][g] = 0.f;
#pragma unroll
            for (int s = 0; s < 32 / 4; ++s) {
                const int c = warp * 32 + s * 4 + gi;
                const uint2 bm = bm_s[c];
                unsigned short coef[G];
                load_coef<G>(qs + c * G, coef);
                tile_step<G>(bm.y, bm.x, val + of[c], sel, mh, ml, coef, acc_s);
            }
            // fold two lane groups (same tokens, other channels), the rest meets in partial planes
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int g = 0; g < G; ++g) acc_s[t][g] += __shfl_xor_sync(kFull, acc_s[t][g], 16);
            if (gi < kGroupsPerWarp) {
                float* dst = spart + (static_cast<size_t>(warp * kGroupsPerWarp + gi) * G) * 64 + kb * 8;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    *reinterpret_cast<float4*>(dst + g * 64) = make_float4(acc_s[0][g], acc_s[1][g], acc_s[2][g], acc_s[3][g]);
                    *reinterpret_cast<float4*>(dst + g * 64 + 4) = make_float4(acc_s[4][g], acc_s[5][g], acc_s[6][g], acc_s[7][g]);
                }
            }
            __syncthreads();
            for (int g = warp; g < G; g += kWarps) {
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int pl = 0; pl < kPlanes; ++pl) {
                    const float2 t = *reinterpret_cast<const float2*>(spart + (static_cast<size_t>(pl) * G + g) * 64 + 2 * lane);
                    s0 += t.x;
                    s1 += t.y;
                }
                *reinterpret_cast<__half2*>(p.s_out + (static_cast<int64_t>(hq) * G + g) * p.s_stride +
                                            static_cast<int64_t>(blk0 + i) * 64 + 2 * lane) = __floats2half2_rn(s0, s1);
            }
            if (i + 1 < nb) store_offsets(i + 1);
        } else {
            // p comes from the caller: warp j loads heads j, j+4, ...; lane takes tokens 2*lane, 2*lane+1
            for (int g = warp; g < G; g += kWarps) {
                const unsigned pv = *reinterpret_cast<const unsigned*>(
                    p.p_in + (static_cast<int64_t>(hq) * G + g) * p.p_stride + static_cast<int64_t>(blk0 + i) * 64 + 2 * lane);
                ps[(2 * lane) * G + g] = pv & 0xffffu;
                ps[(2 * lane + 1) * G + g] = pv >> 16;
            }
            if (i + 1 < nb) store_offsets(i + 1);
            __syncthreads();
            const int half_id = gi & 1, par = gi >> 1;
#pragma unroll
            for (int s = 0; s < 16 / 2; ++s) {
                const int t = warp * 16 + s * 2 + par;
                const int tile = half_id * 64 + t;
                const uint2 bm = bm_s[tile];
                unsigned short coef[G];
                load_coef<G>(ps + t * G, coef);
                tile_step<G>(bm.y, bm.x, val + of[tile], sel, mh, ml, coef, acc_o);
            }
        }
    }

    if (timed_out) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_TIMEOUT);
        return;
    }
    if (MODE == MODE_KEY) return;

    // ---- VALUE epilogue: join token parities (lanes 16 apart), then the 4 warps, and write the partial
    __syncthreads();
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int g = 0; g < G; ++g) acc_o[t][g] += __shfl_xor_sync(kFull, acc_o[t][g], 16);
    float* red = spart;   // [warp][G][128]
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
    for (int idx = tid; idx < G * kD; idx += kThreads) {
        const int g = idx / kD, c = idx % kD;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) s += red[(static_cast<size_t>(w) * G + g) * kD + c];
        rec[g * kPartialStride + c] = s;
    }
}

// Merges the split partials of one q head: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
// (normalise = 1) or the plain sum of O_s (normalise = 0).  One CTA per q head, 128 threads.
__global__ void __launch_bounds__(128) combine_kernel(const float* ws, int nrec, int G, int normalise,
                                                      __half* out, int64_t out_stride) {
    // weight of each record, computed once per CTA (records in chunks of 128), then every thread sums
    // its channel over the records with independent, unrolled loads
    __shared__ float w_s[128];
    __shared__ float red_s[8];
    const int bq = blockIdx.x, h = bq / G, g = bq % G, c = threadIdx.x;
    const float* base = ws + ((static_cast<int64_t>(h) * nrec) * G + g) * kPartialStride;
    const int64_t step = static_cast<int64_t>(G) * kPartialStride;
    float M = -INFINITY;
    if (normalise) {
        for (int s = c; s < nrec; s += 128) M = fmaxf(M, base[s * step + kPartM]);
#pragma unroll
        for (int d = 16; d; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
        if ((c & 31) == 0) red_s[c >> 5] = M;
        __syncthreads();
        M = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
    }
    float o = 0.f, l = 0.f;
    for (int s0 = 0; s0 < nrec; s0 += 128) {
        const int n = min(128, nrec - s0);
        float wl = 0.f;
        if (c < n) {
            float w = 1.f;
            if (normalise) {
                const float ms = base[(s0 + c) * step + kPartM];
                w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
                wl = w * base[(s0 + c) * step + kPartL];
            }
            w_s[c] = w;
        }
#pragma unroll
        for (int d = 16; d; d >>= 1) wl += __shfl_xor_sync(0xffffffffu, wl, d);
        __syncthreads();                       // w_s written; red_s (max) consumed by everyone
        if ((c & 31) == 0) red_s[4 + (c >> 5)] = wl;
        const float* rec = base + s0 * step + c;
        int s = 0;
        for (; s + 8 <= n; s += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = rec[(s + u) * step];
#pragma unroll
            for (int u = 0; u < 8; ++u) o += w_s[s + u] * v[u];
        }
        for (; s < n; ++s) o += w_s[s] * rec[s * step];
        __syncthreads();                       // partial l sums written; w_s free for the next chunk
        l += red_s[4] + red_s[5] + red_s[6] + red_s[7];
    }
    if (normalise) o = (l > 0.f) ? o / l : 0.f;
    out[bq * out_stride + c] = __float2half_rn(o);
}

// ---------------------------------------------------------------------------- host side
template <int G, int MODE>
static int launch_spmv(const DecodeParams& p, int n_kv_heads, int grid_x, cudaStream_t s) {
    const SmemLayout<G> lay(p.cap);
    static size_t configured[64] = {0};   // largest dynamic shared memory size opted into so far, per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MFAR_ERR_LAUNCH;
    if (lay.total > configured[dev]) {
        if (cudaFuncSetAttribute(spmv_kernel<G, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(lay.total)) != cudaSuccess)
            return MFAR_ERR_LAUNCH;
        configured[dev] = lay.total;
    }
    spmv_kernel<G, MODE><<<dim3(grid_x, n_kv_heads), kThreads, lay.total, s>>>(p);
    return launch_status();
}

template <int MODE>
static int dispatch_spmv(const DecodeParams& p, int G, int n_kv_heads, int grid_x, cudaStream_t s) {
    switch (G) {
        case 1: return launch_spmv<1, MODE>(p, n_kv_heads, grid_x, s);
        case 2: return launch_spmv<2, MODE>(p, n_kv_heads, grid_x, s);
        case 4: return launch_spmv<4, MODE>(p, n_kv_heads, grid_x, s);
        default: return MFAR_ERR_ARG;
    }
}

// 8 query heads per kv head need 64 accumulators per lane and spill; they run as two CTAs of 4 query heads that
// read the same kv head (the second read hits L2).  Their partial records lie in the
// [kv head * 2 + half][record][4] layout, which the combine kernel reads with G = 4.
template <int MODE>
static int launch_spmv8(const DecodeParams& p, int n_kv_heads, cudaStream_t s) {
    DecodeParams p2 = p;
    p2.kv_share = 2;
    return launch_spmv<4, MODE>(p2, 2 * n_kv_heads, p.nsplit, s);
}

static int pick_cap(int stage_halves) {
    int cap = stage_halves <= 0 ? 8192 : stage_halves;
    if (cap > 8192) cap = 8192;
    return (cap + 7) & ~7;
}

static int check_sparse(const void* bmp, const void* acc, const void* nz, int64_t bmp_hs, int64_t nz_hs) {
    if (!bmp || !acc || !nz) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(bmp) & 15) || (bmp_hs & 1) || (reinterpret_cast<uintptr_t>(nz) & 15) || (nz_hs & 7) ||
        (reinterpret_cast<uintptr_t>(acc) & 3))
        return MFAR_ERR_ALIGN;
    return MFAR_OK;
}

int launch_combine(const float* ws, int nrec, int G, int normalise, void* out, int64_t out_stride, int n_q_heads,
                   cudaStream_t s) {
    combine_kernel<<<n_q_heads, 128, 0, s>>>(ws, nrec, G, normalise, static_cast<__half*>(out), out_stride);
    return launch_status();
}

}  // namespace mfar

using namespace mfar;

// Split count of the block kernels: the fitted cost model of decode_common.cuh, within the staging limit.
static int block_split(int n_kv_heads, int nblk, int hint) {
    if (nblk <= 0) return 0;
    const int min_ns = (nblk + kMaxBlocksPerSplit - 1) / kMaxBlocksPerSplit;
    int ns = hint > 0 ? hint : model_split_count(n_kv_heads, nblk, min_ns, 128, device_sm_count());
    if (ns < min_ns) ns = min_ns;
    if (ns > nblk) ns = nblk;
    if (ns < 1) ns = 1;
    const int bps = (nblk + ns - 1) / ns;
    return (nblk + bps - 1) / bps;   // no empty splits
}

extern "C" int mfar_decode_plan(int n_kv_heads, int n_tokens, int window, int nsplit_hint, int* nsplit_out,
                                size_t* workspace_bytes, int group) {
    if (n_kv_heads <= 0 || n_tokens < 0 || (n_tokens % 64) || window < 0 || group <= 0) return MFAR_ERR_ARG;
    const int nblk = n_tokens / 64;
    const int ns = block_split(n_kv_heads, nblk, nsplit_hint);
    if (nsplit_out) *nsplit_out = ns;
    if (workspace_bytes)
        *workspace_bytes = counters_bytes(n_kv_heads) +
                           static_cast<size_t>(n_kv_heads) * (ns + 1) * group * kPartialStride * sizeof(float) + 16;
    return MFAR_OK;
}

static int decode_attention_fp16_impl(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, int64_t k_bmp_head_stride, const int32_t* k_accum, int64_t k_acc_head_stride,
    const void* k_nz, const int32_t* k_nz_offset, int64_t k_nz_head_stride, int64_t k_nz_extent,
    const int64_t* v_bitmaps, int64_t v_bmp_head_stride, const int32_t* v_accum, int64_t v_acc_head_stride,
    const void* v_nz, const int32_t* v_nz_offset, int64_t v_nz_head_stride, int64_t v_nz_extent,
    int n_tokens, const int32_t* n_tokens_dev, const void* k_window, const void* v_window, int64_t win_head_stride,
    int64_t win_token_stride, int window, const int32_t* window_len_dev, float softmax_scale, void* out,
    int64_t out_stride, void* workspace, size_t workspace_bytes, int nsplit, int stage_halves,
    uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens < 0 || (n_tokens % 64) || window < 0) return MFAR_ERR_ARG;
    if (n_tokens == 0 && window == 0) return MFAR_ERR_ARG;
    if (group != 1 && group != 2 && group != 4 && group != 8) return MFAR_ERR_ARG;
    if (!q || !out || !workspace || k_nz_extent < 0 || v_nz_extent < 0) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(q) & 3) || (q_stride & 1)) return MFAR_ERR_ALIGN;
    if (window > 0 && (!k_window || !v_window)) return MFAR_ERR_ARG;
    if (window > 0 && ((reinterpret_cast<uintptr_t>(k_window) & 15) || (reinterpret_cast<uintptr_t>(v_window) & 15) ||
                       (win_head_stride & 7) || (win_token_stride & 7)))
        return MFAR_ERR_ALIGN;
    if (n_tokens > 0) {
        int r = check_sparse(k_bitmaps, k_accum, k_nz, k_bmp_head_stride, k_nz_head_stride);
        if (r) return r;
        r = check_sparse(v_bitmaps, v_accum, v_nz, v_bmp_head_stride, v_nz_head_stride);
        if (r) return r;
    }
    int ns = 0;
    size_t need = 0;
    int r = mfar_decode_plan(n_kv_heads, n_tokens, window, nsplit, &ns, &need, group);
    if (r) return r;
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return MFAR_ERR_WORKSPACE;

    DecodeParams p{};
    p.k = Sparse{reinterpret_cast<const unsigned long long*>(k_bitmaps), k_accum, static_cast<const __half*>(k_nz),
                 k_nz_offset, k_bmp_head_stride, k_acc_head_stride, k_nz_head_stride, k_nz_extent};
    p.v = Sparse{reinterpret_cast<const unsigned long long*>(v_bitmaps), v_accum, static_cast<const __half*>(v_nz),
                 v_nz_offset, v_bmp_head_stride, v_acc_head_stride, v_nz_head_stride, v_nz_extent};
    p.q = static_cast<const __half*>(q);
    p.q_stride = q_stride;
    p.kwin = static_cast<const __half*>(k_window);
    p.vwin = static_cast<const __half*>(v_window);
    p.win_hs = win_head_stride;
    p.win_ts = win_token_stride;
    p.W = window;
    p.W_dev = window_len_dev;
    p.L_dev = n_tokens_dev;
    p.nblk = n_tokens / 64;
    p.cap = pick_cap(stage_halves);
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    // more kv heads than counters: the records are merged by a second launch instead
    p.counters = n_kv_heads <= kMaxCountedHeads ? static_cast<unsigned*>(workspace) : nullptr;
    p.ws = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + counters_bytes(n_kv_heads));
    p.out = static_cast<__half*>(out);
    p.out_stride = out_stride;
    p.dev_status = dev_status;
    p.nsplit = ns;
    p.bps = ns > 0 ? (p.nblk + ns - 1) / ns : 0;
    p.nrec = ns + (window > 0 ? 1 : 0);
    p.rec_group = group;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    r = launch_decode_attn(p, group, n_kv_heads, p.nrec, s);
    if (r || p.counters) return r;
    return launch_combine(p.ws, p.nrec, group, 1, out, out_stride, n_kv_heads * group, s);
}

extern "C" int mfar_decode_attention_fp16(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, int64_t k_bmp_head_stride, const int32_t* k_accum, int64_t k_acc_head_stride,
    const void* k_nz, const int32_t* k_nz_offset, int64_t k_nz_head_stride, int64_t k_nz_extent,
    const int64_t* v_bitmaps, int64_t v_bmp_head_stride, const int32_t* v_accum, int64_t v_acc_head_stride,
    const void* v_nz, const int32_t* v_nz_offset, int64_t v_nz_head_stride, int64_t v_nz_extent,
    int n_tokens, const void* k_window, const void* v_window, int64_t win_head_stride, int64_t win_token_stride,
    int window, const int32_t* window_len_dev, float softmax_scale, void* out, int64_t out_stride, void* workspace,
    size_t workspace_bytes, int nsplit, int stage_halves, uint32_t* dev_status, void* stream) {
    return decode_attention_fp16_impl(q, q_stride, n_kv_heads, group, k_bitmaps, k_bmp_head_stride, k_accum,
                                      k_acc_head_stride, k_nz, k_nz_offset, k_nz_head_stride, k_nz_extent, v_bitmaps,
                                      v_bmp_head_stride, v_accum, v_acc_head_stride, v_nz, v_nz_offset, v_nz_head_stride,
                                      v_nz_extent, n_tokens, nullptr, k_window, v_window, win_head_stride,
                                      win_token_stride, window, window_len_dev, softmax_scale, out, out_stride,
                                      workspace, workspace_bytes, nsplit, stage_halves, dev_status, stream);
}

extern "C" int mfar_decode_attention_fp16_dyn(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, int64_t k_bmp_head_stride, const int32_t* k_accum, int64_t k_acc_head_stride,
    const void* k_nz, const int32_t* k_nz_offset, int64_t k_nz_head_stride, int64_t k_nz_extent,
    const int64_t* v_bitmaps, int64_t v_bmp_head_stride, const int32_t* v_accum, int64_t v_acc_head_stride,
    const void* v_nz, const int32_t* v_nz_offset, int64_t v_nz_head_stride, int64_t v_nz_extent,
    int max_tokens, const int32_t* n_tokens_dev, const void* k_window, const void* v_window, int64_t win_head_stride,
    int64_t win_token_stride, int window, const int32_t* window_len_dev, float softmax_scale, void* out,
    int64_t out_stride, void* workspace, size_t workspace_bytes, int nsplit, int stage_halves,
    uint32_t* dev_status, void* stream) {
    if (!n_tokens_dev) return MFAR_ERR_ARG;
    return decode_attention_fp16_impl(q, q_stride, n_kv_heads, group, k_bitmaps, k_bmp_head_stride, k_accum,
                                      k_acc_head_stride, k_nz, k_nz_offset, k_nz_head_stride, k_nz_extent, v_bitmaps,
                                      v_bmp_head_stride, v_accum, v_acc_head_stride, v_nz, v_nz_offset, v_nz_head_stride,
                                      v_nz_extent, max_tokens, n_tokens_dev, k_window, v_window, win_head_stride,
                                      win_token_stride, window, window_len_dev, softmax_scale, out, out_stride,
                                      workspace, workspace_bytes, nsplit, stage_halves, dev_status, stream);
}

extern "C" int mfar_key_scores_fp16(const void* q, int64_t q_stride, int n_kv_heads, int group,
                                    const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* accum,
                                    int64_t acc_head_stride, const void* nz, const int32_t* nz_offset,
                                    int64_t nz_head_stride, int64_t nz_extent, int n_tokens, void* scores,
                                    int64_t scores_stride, int stage_halves, uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens < 0 || (n_tokens % 64) || nz_extent < 0) return MFAR_ERR_ARG;
    if (group != 1 && group != 2 && group != 4 && group != 8) return MFAR_ERR_ARG;
    if (n_tokens == 0) return MFAR_OK;
    if (!q || !scores) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(scores) & 3) || (scores_stride & 1)) return MFAR_ERR_ALIGN;
    int r = check_sparse(bitmaps, accum, nz, bmp_head_stride, nz_head_stride);
    if (r) return r;
    DecodeParams p{};
    p.k = Sparse{reinterpret_cast<const unsigned long long*>(bitmaps), accum, static_cast<const __half*>(nz), nz_offset,
                 bmp_head_stride, acc_head_stride, nz_head_stride, nz_extent};
    p.q = static_cast<const __half*>(q);
    p.q_stride = q_stride;
    p.nblk = n_tokens / 64;
    // enough CTAs to fill the machine, a few blocks each so that the ring has something to overlap
    int ns = (device_sm_count() * 6 + n_kv_heads - 1) / n_kv_heads;
    const int min_ns = (p.nblk + kMaxBlocksPerSplit - 1) / kMaxBlocksPerSplit;
    if (ns > (p.nblk + 3) / 4) ns = (p.nblk + 3) / 4;
    if (ns < min_ns) ns = min_ns;
    if (ns < 1) ns = 1;
    p.bps = (p.nblk + ns - 1) / ns;
    p.nsplit = (p.nblk + p.bps - 1) / p.bps;
    p.cap = pick_cap(stage_halves);
    p.s_out = static_cast<__half*>(scores);
    p.s_stride = scores_stride;
    p.dev_status = dev_status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (group == 8) return launch_spmv8<MODE_KEY>(p, n_kv_heads, s);
    return dispatch_spmv<MODE_KEY>(p, group, n_kv_heads, p.nsplit, s);
}

extern "C" int mfar_value_output_fp16(const void* probs, int64_t probs_stride, int n_kv_heads, int group,
                                      const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* accum,
                                      int64_t acc_head_stride, const void* nz, const int32_t* nz_offset,
                                      int64_t nz_head_stride, int64_t nz_extent, int n_tokens, void* out,
                                      int64_t out_stride, void* workspace, size_t workspace_bytes, int nsplit,
                                      int stage_halves, uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens <= 0 || (n_tokens % 64) || nz_extent < 0) return MFAR_ERR_ARG;
    if (group != 1 && group != 2 && group != 4 && group != 8) return MFAR_ERR_ARG;
    if (!probs || !out || !workspace) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(probs) & 3) || (probs_stride & 1)) return MFAR_ERR_ALIGN;
    int r = check_sparse(bitmaps, accum, nz, bmp_head_stride, nz_head_stride);
    if (r) return r;
    int ns = 0;
    size_t need = 0;
    r = mfar_decode_plan(n_kv_heads, n_tokens, 0, nsplit, &ns, &need, group);
    if (r) return r;
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return MFAR_ERR_WORKSPACE;
    DecodeParams p{};
    p.v = Sparse{reinterpret_cast<const unsigned long long*>(bitmaps), accum, static_cast<const __half*>(nz), nz_offset,
                 bmp_head_stride, acc_head_stride, nz_head_stride, nz_extent};
    p.nblk = n_tokens / 64;
    p.nsplit = ns;
    p.nrec = ns;
    p.bps = (p.nblk + ns - 1) / ns;
    p.cap = pick_cap(stage_halves);
    p.p_in = static_cast<const __half*>(probs);
    p.p_stride = probs_stride;
    p.ws = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + counters_bytes(n_kv_heads));
    p.dev_status = dev_status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    r = group == 8 ? launch_spmv8<MODE_VALUE>(p, n_kv_heads, s) : dispatch_spmv<MODE_VALUE>(p, group, n_kv_heads, ns, s);
    if (r) return r;
    return launch_combine(p.ws, ns, group == 8 ? 4 : group, 0, out, out_stride, n_kv_heads * group, s);
}
