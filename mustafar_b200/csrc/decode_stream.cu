// Fused decode attention, "stream" kernel: no CTA-wide barrier inside the block loop.
//
// A CTA of 4 warps walks a range of 64-token blocks of ONE kv head for all G query heads.  The
// block's bitmaps and packed values of K and V sit in a 2-stage shared-memory ring filled by 1-D
// bulk copies (cp.async.bulk + mbarrier, no multicast).
//   refill        : the warp that is LAST to finish a block (a shared-memory counter tells) issues
//                   the bulk copies of the block two ahead into the stage it has just freed,
//                   converts that block's 2 x 128 accum entries to shared-memory offsets and flips
//                   the stage's "ready" barrier;
//   warp w        : owns tokens 16w .. 16w+15 of EVERY block, in both phases, so scores,
//                   softmax state and probabilities never leave the warp:
//       K phase   2 lanes per tile (the two bitmap bytes that cover the warp's 16 tokens),
//                 16 tiles (channels) per step, 8 steps; the 16 per-channel partials of a score
//                 meet through a warp-private shared-memory patch;
//       softmax   online max / sum per head over the warp's own tokens (a warp is an independent
//                 split-KV stream, merged with the other three at the end of the CTA);
//       V phase   8 lanes per tile (one byte = 8 channels each), 2 tokens x 2 halves per step.
// Tile decode: rank of the lane's first position = popc of the bitmap bits before its byte, every
// set bit consumes the next packed half; multiply-accumulate in fp32 for all G heads, either with
// fp32 coefficients or (MIXED) with fp16 coefficients in one mixed-precision FMA.
#include <type_traits>

#include "decode_common.cuh"

namespace mfar {

constexpr int kStWarps = 4;                 // consumer warps
constexpr int kStThreads = kStWarps * 32;
#ifndef MFAR_ST_STAGES
#define MFAR_ST_STAGES 2
#endif
#ifndef MFAR_ST_MINB
#define MFAR_ST_MINB 4
#endif
constexpr int kStStages = MFAR_ST_STAGES;
constexpr int kStMaxBlocks = 512;

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int G, bool MIXED>
struct StLayout {
    using coef_t = typename std::conditional<MIXED, unsigned short, float>::type;
    static constexpr int ROW = 8 * G + 4;    // floats per lane row of the K-phase patch (padded: conflict free)
    size_t stages, bars, q, red, ps, mstate, kblk, vblk, total;
    size_t s_kbm, s_vbm, s_koff, s_voff, s_kval, s_vval, stage;
    __host__ __device__ explicit StLayout(int cap) {
        const size_t val = (static_cast<size_t>(cap) + kSlackHalves) * 2;
        s_kbm = 0; s_vbm = 1024; s_koff = 2048; s_voff = 2560; s_kval = 3072; s_vval = s_kval + val;
        stage = s_vval + val;
        size_t o = 0;
        stages = o; o += kStStages * stage;
        bars = o;   o += 32 * kStStages;   // full + ready barriers and the done counter of every stage
        q = o;      o += kD * G * sizeof(coef_t);
        red = o;    o += static_cast<size_t>(kStWarps) * 32 * ROW * 4;     // reused by the epilogue
        ps = o;     o += kStWarps * 16 * G * sizeof(coef_t) + 64;
        mstate = o; o += 2 * kStWarps * G * 4 + 64;
        kblk = o;   o += (kStMaxBlocks + 4) * 4;
        vblk = o;   o += (kStMaxBlocks + 4) * 4;
        total = (o + 15) & ~static_cast<size_t>(15);
    }
};

template <int G, bool MIXED>
__global__ void __launch_bounds__(kStThreads, MFAR_ST_MINB) decode_stream_kernel(DecodeParams p) {
    using L = StLayout<G, MIXED>;
    using coef_t = typename L::coef_t;
    constexpr int ROW = L::ROW;
    constexpr int HP = G >= 2 ? G / 2 : 1;          // heads a lane owns in the softmax

    extern __shared__ __align__(128) unsigned char smem[];
    const L lay(p.cap);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + lay.bars);
    unsigned long long* bar_full = bars;                 // [kStStages] bulk copies landed
    unsigned long long* bar_ready = bars + kStStages;    // [kStStages] ... and offsets converted
    unsigned* done_cnt = reinterpret_cast<unsigned*>(bars + 2 * kStStages);   // [kStStages] warps done with the stage
    static_assert(2 * kStStages * 8 + kStStages * 4 <= 32 * kStStages, "barrier area");
    coef_t* qs = reinterpret_cast<coef_t*>(smem + lay.q);           // [128][G]
    float* red = reinterpret_cast<float*>(smem + lay.red);          // [warp][lane][ROW]
    coef_t* ps = reinterpret_cast<coef_t*>(smem + lay.ps);          // [warp][16][G]
    float* mstate = reinterpret_cast<float*>(smem + lay.mstate);    // m[warp][G], l[warp][G]
    int* kblk = reinterpret_cast<int*>(smem + lay.kblk);
    int* vblk = reinterpret_cast<int*>(smem + lay.vblk);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.y, split = blockIdx.x;
    const int blk0 = split * p.bps;
    const int nb = max(0, min(p.bps, p.nblk - blk0));

    for (int i = tid; i < kD * G; i += kStThreads) {
        const int c = i / G, g = i % G;
        store_coef(&qs[i], __half2float(p.q[(static_cast<int64_t>(h) * G + g) * p.q_stride + c]));
    }
    const int* kacc = p.k.acc + h * p.k.acc_hs;
    const int* vacc = p.v.acc + h * p.v.acc_hs;
    for (int i = tid; i <= nb; i += kStThreads) {
        kblk[i] = kacc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
        vblk[i] = vacc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
    }
    if (tid == 0) {
        for (int s = 0; s < kStStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_ready[s], 1);
            done_cnt[s] = 0;
        }
        mbar_fence_init();
    }
    __syncthreads();

    const __half* knz = p.k.nz + (p.k.nz_off ? 8ll * p.k.nz_off[h] : h * p.k.nz_hs);
    const __half* vnz = p.v.nz + (p.v.nz_off ? 8ll * p.v.nz_off[h] : h * p.v.nz_hs);
    const unsigned capb = static_cast<unsigned>(p.cap) * 2u;

    // Brings block i of this split into stage i % kStStages; called by ONE whole warp once every
    // warp is done with the block that used the stage before.
    auto refill = [&](int i) {
        const int s = i % kStStages;
        unsigned char* st = smem + lay.stages + static_cast<size_t>(s) * lay.stage;
        const int64_t tile0 = static_cast<int64_t>(blk0 + i) * kTilesPerBlock;
        int ko[4], vo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            ko[e] = kacc[tile0 + lane + 32 * e];
            vo[e] = vacc[tile0 + lane + 32 * e];
        }
        if (lane == 0) {
            const long long dk = (static_cast<long long>(kblk[i + 1]) - kblk[i]) * 4;
            const long long dv = (static_cast<long long>(vblk[i + 1]) - vblk[i]) * 4;
            const bool bad = dk < 0 || dk > capb || dv < 0 || dv > capb || kblk[i] < 0 || vblk[i] < 0;
            const unsigned kbytes = bad ? 0u : (static_cast<unsigned>(dk) & ~15u);
            const unsigned vbytes = bad ? 0u : (static_cast<unsigned>(dv) & ~15u);
            if (bad && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_BADMETA);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&bar_full[s], 2048 + kbytes + vbytes);
            bulk_g2s(st + lay.s_kbm, p.k.bmp + h * p.k.bmp_hs + tile0, 1024, &bar_full[s]);
            bulk_g2s(st + lay.s_vbm, p.v.bmp + h * p.v.bmp_hs + tile0, 1024, &bar_full[s]);
            if (kbytes) bulk_g2s(st + lay.s_kval, knz + 2ll * kblk[i], kbytes, &bar_full[s]);
            if (vbytes) bulk_g2s(st + lay.s_vval, vnz + 2ll * vblk[i], vbytes, &bar_full[s]);
        }
        unsigned* koff = reinterpret_cast<unsigned*>(st + lay.s_koff);
        unsigned* voff = reinterpret_cast<unsigned*>(st + lay.s_voff);
        const unsigned lim = static_cast<unsigned>(p.cap);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            koff[lane + 32 * e] = min(static_cast<unsigned>(2 * (ko[e] - kblk[i])), lim);
            voff[lane + 32 * e] = min(static_cast<unsigned>(2 * (vo[e] - vblk[i])), lim);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_ready[s]);
    };
    if (warp < kStStages && warp < nb) refill(warp);     // the first blocks: one warp each

    bool timed_out = false;
    float acc_o[8][G];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int g = 0; g < G; ++g) acc_o[i][g] = 0.f;
    float m_run[HP], l_run[HP];
#pragma unroll
    for (int j = 0; j < HP; ++j) { m_run[j] = -INFINITY; l_run[j] = 0.f; }

    {
        const int gi = lane >> 3, kb = lane & 7;
        unsigned selV, mhV, mlV, selK, mhK, mlK;
        lane_byte_constants(kb, selV, mhV, mlV);
        lane_byte_constants(2 * warp + (lane & 1), selK, mhK, mlK);
        const int slot = lane >> 1;                         // K phase: which of the 16 tiles of a step
        float* myrow = red + (static_cast<size_t>(warp) * 32 + lane) * ROW;
        const int tt = lane >> 1, hb = (G >= 2) ? (lane & 1) * HP : 0;   // softmax: token and first head of this lane
        const float* rsrc = red + (static_cast<size_t>(warp) * 32 + (tt >> 3)) * ROW + (tt & 7) * G + hb;
        coef_t* myps = ps + (static_cast<size_t>(warp) * 16) * G;

        for (int i = 0; i < nb; ++i) {
            const int s = i % kStStages, n = i / kStStages;
            const unsigned char* st = smem + lay.stages + static_cast<size_t>(s) * lay.stage;
            if (!mbar_wait(&bar_ready[s], n & 1) || !mbar_wait(&bar_full[s], n & 1)) timed_out = true;
            timed_out = __any_sync(kFull, timed_out);
            if (timed_out) break;
            const uint2* kbm = reinterpret_cast<const uint2*>(st + lay.s_kbm);
            const uint2* vbm = reinterpret_cast<const uint2*>(st + lay.s_vbm);
            const unsigned* koff = reinterpret_cast<const unsigned*>(st + lay.s_koff);
            const unsigned* voff = reinterpret_cast<const unsigned*>(st + lay.s_voff);
            const unsigned short* kval = reinterpret_cast<const unsigned short*>(st + lay.s_kval);
            const unsigned short* vval = reinterpret_cast<const unsigned short*>(st + lay.s_vval);

            // ---------------------------------------------------- K phase: 16 tokens x 128 channels
            {
                float acc_s[8][G];
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int g = 0; g < G; ++g) acc_s[t][g] = 0.f;
#pragma unroll 4
                for (int s8 = 0; s8 < 8; ++s8) {
                    const int c = s8 * 16 + slot;
                    const uint2 bm = kbm[c];
                    coef_t coef[G];
                    load_coef<G>(qs + c * G, coef);
                    tile_step<G>(bm.y, bm.x, kval + koff[c], selK, mhK, mlK, coef, acc_s);
                }
                // row layout [token i][head g]
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    if constexpr (G % 4 == 0) {
#pragma unroll
                        for (int g = 0; g < G; g += 4)
                            *reinterpret_cast<float4*>(myrow + t * G + g) = make_float4(acc_s[t][g], acc_s[t][g + 1], acc_s[t][g + 2], acc_s[t][g + 3]);
                    } else {
#pragma unroll
                        for (int g = 0; g < G; ++g) myrow[t * G + g] = acc_s[t][g];
                    }
                }
            }
            __syncwarp();

            // ---------------------------------------------------- scores of (token tt, heads hb..) -> probabilities
            float a_own[HP];
            {
                float sc[HP];
#pragma unroll
                for (int j = 0; j < HP; ++j) sc[j] = 0.f;
#pragma unroll
                for (int sl = 0; sl < 16; ++sl) {
                    const float* src = rsrc + static_cast<size_t>(2 * sl) * ROW;
                    if constexpr (HP == 4) {
                        const float4 t = *reinterpret_cast<const float4*>(src);
                        sc[0] += t.x; sc[1] += t.y; sc[2] += t.z; sc[3] += t.w;
                    } else if constexpr (HP == 2) {
                        const float2 t = *reinterpret_cast<const float2*>(src);
                        sc[0] += t.x; sc[1] += t.y;
                    } else {
                        sc[0] += src[0];
                    }
                }
#pragma unroll
                for (int j = 0; j < HP; ++j) {
                    const float sv = sc[j] * p.scale_log2;
                    float mx = sv;   // max over the warp's 16 tokens: lanes of equal parity
#pragma unroll
                    for (int d = 2; d < 32; d <<= 1) mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, d));
                    const float m_new = fmaxf(m_run[j], mx);
                    a_own[j] = fast_exp2(m_run[j] - m_new);
                    const float pr = round_like(myps, fast_exp2(sv - m_new));
                    l_run[j] = l_run[j] * a_own[j] + pr;
                    m_run[j] = m_new;
                    store_coef(&myps[tt * G + hb + j], pr);
                }
            }
            // every lane needs the rescale factor of all G heads: its own HP, the partner lane's HP
            {
                float a[G];
                bool any = false;
                float other[HP];
#pragma unroll
                for (int j = 0; j < HP; ++j) other[j] = __shfl_xor_sync(kFull, a_own[j], 1);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const bool mine = (G < 2) || ((lane & 1) == (g / HP));
                    a[g] = mine ? a_own[g % HP] : other[g % HP];
                }
#pragma unroll
                for (int g = 0; g < G; ++g) any |= (a[g] != 1.f);
                if (any) {
#pragma unroll
                    for (int t = 0; t < 8; ++t)
#pragma unroll
                        for (int g = 0; g < G; ++g) acc_o[t][g] *= a[g];
                }
            }
            __syncwarp();

            // ---------------------------------------------------- V phase: the warp's 16 tokens x 128 channels
            {
                const int half_id = gi & 1, par = gi >> 1;
#pragma unroll 4
                for (int s8 = 0; s8 < 8; ++s8) {
                    const int tl = s8 * 2 + par;                  // token inside the warp's 16
                    const int tile = half_id * 64 + warp * 16 + tl;
                    const uint2 bm = vbm[tile];
                    coef_t coef[G];
                    load_coef<G>(myps + tl * G, coef);
                    tile_step<G>(bm.y, bm.x, vval + voff[tile], selV, mhV, mlV, coef, acc_o);
                }
            }
            // release the stage; the last of the 4 warps to get here refills it with block i + kStStages
            __syncwarp();
            unsigned last = 0;
            if (lane == 0) {
                __threadfence_block();
                last = (atomicAdd(&done_cnt[s], 1u) == kStWarps - 1) ? 1u : 0u;
                if (last) {
                    done_cnt[s] = 0;
                    __threadfence_block();
                }
            }
            last = __shfl_sync(kFull, last, 0);
            if (last && i + kStStages < nb) refill(i + kStStages);
        }
    }

    // ---- epilogue: the 4 warps are 4 split-KV streams with their own running max
    timed_out = __syncthreads_or(timed_out);
    if (timed_out) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_TIMEOUT);
        return;
    }
    float* m_s = mstate;                    // [warp][G]
    float* l_s = mstate + kStWarps * G;     // [warp][G]
    {
        const int hb = (G >= 2) ? (lane & 1) * HP : 0;
#pragma unroll
        for (int j = 0; j < HP; ++j) {
            float l = l_run[j];
#pragma unroll
            for (int d = 2; d < 32; d <<= 1) l += __shfl_xor_sync(kFull, l, d);
            if (lane < 2 && (G >= 2 || lane == 0)) {
                m_s[warp * G + hb + j] = m_run[j];
                l_s[warp * G + hb + j] = l;
            }
        }
    }
    __syncthreads();
    {
        const int gi = lane >> 3, kb = lane & 7;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kStWarps; ++w) M = fmaxf(M, m_s[w * G + g]);
            const float mb = m_s[warp * G + g];
            const float wgt = (mb == -INFINITY) ? 0.f : fast_exp2(mb - M);
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float v = acc_o[j][g] * wgt;
                f[j] = v + __shfl_xor_sync(kFull, v, 16);
            }
            if (lane < 16) {
                float* d = red + (static_cast<size_t>(warp) * G + g) * kD + (gi & 1) * 64 + kb * 8;
                *reinterpret_cast<float4*>(d) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(d + 4) = make_float4(f[4], f[5], f[6], f[7]);
            }
        }
    }
    __syncthreads();
    const int nrec = p.nsplit + (p.W > 0 ? 1 : 0);
    float* rec = p.ws + ((static_cast<int64_t>(h) * nrec + split) * G) * kPartialStride;
    for (int idx = tid; idx < G * kD; idx += kStThreads) {
        const int g = idx / kD, c = idx % kD;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kStWarps; ++w) sum += red[(static_cast<size_t>(w) * G + g) * kD + c];
        rec[g * kPartialStride + c] = sum;
    }
    if (tid < G) {
        const int g = tid;
        float M = -INFINITY;
        for (int w = 0; w < kStWarps; ++w) M = fmaxf(M, m_s[w * G + g]);
        float l = 0.f;
        for (int w = 0; w < kStWarps; ++w) {
            const float ms = m_s[w * G + g];
            if (ms != -INFINITY) l += l_s[w * G + g] * fast_exp2(ms - M);
        }
        rec[g * kPartialStride + kPartM] = M;
        rec[g * kPartialStride + kPartL] = l;
    }
}

template <int G, bool MIXED>
static int launch_stream(const DecodeParams& p, int n_kv_heads, cudaStream_t s) {
    const StLayout<G, MIXED> lay(p.cap);
    if (lay.total > 227 * 1024) return MFAR_ERR_ARG;
    static size_t configured[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MFAR_ERR_LAUNCH;
    if (lay.total > configured[dev]) {
        if (cudaFuncSetAttribute(decode_stream_kernel<G, MIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(lay.total)) != cudaSuccess)
            return MFAR_ERR_LAUNCH;
        configured[dev] = lay.total;
    }
    decode_stream_kernel<G, MIXED><<<dim3(p.nsplit, n_kv_heads), kStThreads, lay.total, s>>>(p);
    return launch_status();
}

int launch_decode_stream(const DecodeParams& p, int G, int n_kv_heads, bool mixed, cudaStream_t s) {
#define MFAR_ST(GG) \
    case GG: return mixed ? launch_stream<GG, true>(p, n_kv_heads, s) : launch_stream<GG, false>(p, n_kv_heads, s);
    switch (G) {
        MFAR_ST(1)
        MFAR_ST(2)
        MFAR_ST(4)
        MFAR_ST(8)
        default: return MFAR_ERR_ARG;
    }
#undef MFAR_ST
}

int decode_stream_max_blocks() { return kStMaxBlocks; }

}  // namespace mfar
