// Decode attention over the bitmap + packed-fp16 cache.
//
// One kernel template, three modes:
//   ATTN   q.K^T over the compressed tokens, online softmax, P.V, split-KV partials
//          (+ one extra CTA per kv head for the dense recent-token window);
//   KEY    only S = K~ q           (what mustafar_key_formulation returns in row 0);
//   VALUE  only O = V~^T p         (what mustafar_value_formulation returns in row 0).
//
// A CTA (4 warps) walks a range of 64-token blocks of ONE kv head and serves all G
// query heads that share it, so the compressed bytes are read once.  Per block the
// two bitmap arrays (1 KiB each) and the two packed-value ranges are brought into a
// 2-stage shared-memory ring by 1-D bulk copies (cp.async.bulk + mbarrier, issued by
// one thread one block ahead; four CTAs per SM keep ~60 KB in flight).  Tiles are decoded straight from the bitmap:
//   * a lane owns one BYTE of a tile's bitmap = 8 consecutive positions, 8 lanes
//     cover a tile, a warp does 4 tiles per step;
//   * rank of the lane's first position = popc of the bitmap bits before its byte;
//   * position i of the byte: if the bit is set, load the next packed half and
//     multiply-accumulate it in fp32 for all G heads (registers, no dense expansion).
// K phase: lane owns 8 tokens, loops over its warp's 32 channels (a K tile is one
// channel x 64 tokens).  V phase: lane owns 8 channels, loops over its warp's 16
// tokens (a V tile is one token x 64 channels).  Tensor cores are not used.
#include <type_traits>

#include "decode_common.cuh"

namespace mfar {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
#ifndef MFAR_STAGES
#define MFAR_STAGES 2
#endif
constexpr int kStages = MFAR_STAGES;
// K-phase partial planes: (warp, lane group), halved by every shuffle stage that folds two lane groups first
#ifndef MFAR_PLANE_FOLD
#define MFAR_PLANE_FOLD 1
#endif
constexpr int kPlaneFold = MFAR_PLANE_FOLD;                 // 0, 1 or 2
constexpr int kGroupsPerWarp = 4 >> kPlaneFold;
constexpr int kPlanes = kWarps * kGroupsPerWarp;
static_assert(kPlanes * 64 >= kWarps * kD, "the epilogue reuses the score planes as [warp][G][128] floats");
constexpr int kMaxBlocksPerSplit = 256;

// A stage holds, per staged tensor, 1 KiB of bitmaps and cap (+slack) packed halves;
// ATTN stages both K and V, KEY / VALUE only their own.
__host__ __device__ inline size_t stage_bytes(int cap, int mode) {
    return (mode == MODE_ATTN ? 2 : 1) * (1024 + (static_cast<size_t>(cap) + kSlackHalves) * 2);
}

template <int G, int MODE>
struct SmemLayout {
    size_t stages, bars, qs, spart, ps, alpha, koff, voff, kblk, vblk, total;
    // offsets inside a stage
    size_t s_kbm, s_vbm, s_kval, s_vval;
    __host__ __device__ explicit SmemLayout(int cap) {
        s_kbm = 0;
        s_vbm = (MODE == MODE_ATTN) ? 1024 : 0;
        s_kval = (MODE == MODE_ATTN) ? 2048 : 1024;
        s_vval = s_kval + ((MODE == MODE_ATTN) ? (static_cast<size_t>(cap) + kSlackHalves) * 2 : 0);
        size_t o = 0;
        stages = o; o += kStages * stage_bytes(cap, MODE);
        bars = o;   o += 64;
        qs = o;     o += kD * G * 4;
        spart = o;  o += static_cast<size_t>(kPlanes) * G * 64 * 4;
        ps = o;     o += 64 * G * 4;
        alpha = o;  o += 64;
        koff = o;   o += 2 * 128 * 4;
        voff = o;   o += 2 * 128 * 4;
        kblk = o;   o += (kMaxBlocksPerSplit + 4) * 4;
        vblk = o;   o += (kMaxBlocksPerSplit + 4) * 4;
        total = o;
    }
};

#ifndef MFAR_MIN_BLOCKS
#define MFAR_MIN_BLOCKS 4
#endif
#ifndef MFAR_STEP_UNROLL
#define MFAR_STEP_UNROLL 8
#endif
// Ablation switches for timing experiments (never set in a product build: results are then wrong):
//   MFAR_ABL_NOLOAD     only the first kStages blocks are fetched, later iterations reuse the stages
//   MFAR_ABL_NOSOFTMAX  skip the scores -> probabilities section
//   MFAR_ABL_NOSYNC     CTA barriers inside the block loop become warp barriers
#ifdef MFAR_ABL_NOSYNC
#define MFAR_LOOP_SYNC() __syncwarp()
#else
#define MFAR_LOOP_SYNC() __syncthreads()
#endif
#define MFAR_PRAGMA(x) _Pragma(#x)
#define MFAR_UNROLL(n) MFAR_PRAGMA(unroll n)

template <int G, int MODE, bool MIXED>
__global__ void __launch_bounds__(kThreads, MFAR_MIN_BLOCKS) decode_kernel(DecodeParams p) {
    // MIXED: q and the probabilities are held as fp16 and multiplied by the packed halves in one
    // mixed-precision FMA (exact for KEY / VALUE, whose coefficients are fp16 inputs anyway)
    using coef_t = typename std::conditional<MIXED, unsigned short, float>::type;
    extern __shared__ __align__(128) unsigned char smem[];
    const SmemLayout<G, MODE> lay(p.cap);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + lay.bars);
    coef_t* qs = reinterpret_cast<coef_t*>(smem + lay.qs);        // [128][G]
    float* spart = reinterpret_cast<float*>(smem + lay.spart);    // [plane][G][64]
    coef_t* ps = reinterpret_cast<coef_t*>(smem + lay.ps);        // [64][G]
    float* alpha_s = reinterpret_cast<float*>(smem + lay.alpha);  // [G]
    unsigned* koff = reinterpret_cast<unsigned*>(smem + lay.koff);  // [2][128] halves, relative to the block
    unsigned* voff = reinterpret_cast<unsigned*>(smem + lay.voff);
    int* kblk = reinterpret_cast<int*>(smem + lay.kblk);          // block starts (uint32 units) of this split
    int* vblk = reinterpret_cast<int*>(smem + lay.vblk);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // hq numbers the (kv head, group of G query heads) pairs; with kv_share > 1 several of them read the same kv head
    const int hq = blockIdx.y;
    const int h = hq / (p.kv_share > 0 ? p.kv_share : 1);
    const int split = blockIdx.x + p.split_offset;
    const bool is_window = (MODE == MODE_ATTN) && (split == p.nsplit);
    const int gi = lane >> 3, kb = lane & 7;
    unsigned sel, mh, ml;
    lane_byte_constants(kb, sel, mh, ml);

    // the compressed length may live in device memory too (a captured launch keeps working while blocks are
    // appended): p.nblk is then its upper bound, the grid was sized for that bound, and the blocks actually there
    // are dealt out again over the same number of splits (splits past the end write an empty record)
    int nblk = p.nblk, bps = p.bps;
    if (p.L_dev) {
        nblk = max(0, min(*p.L_dev / 64, p.nblk));
        bps = p.nsplit > 0 ? (nblk + p.nsplit - 1) / p.nsplit : 0;
    }
    const int blk0 = is_window ? 0 : split * bps;
    // the window length may live in device memory (so that a captured launch can be replayed while
    // the window grows); p.W is then only its upper bound
    const int W = (is_window && p.W_dev) ? max(0, min(*p.W_dev, p.W)) : p.W;
    int nb = is_window ? (W + 63) / 64 : min(bps, nblk - blk0);
    if (nb < 0) nb = 0;

    // ---- prologue: q to shared memory, block offsets of this split, barriers
    if (MODE != MODE_VALUE) {
        for (int i = tid; i < kD * G; i += kThreads) {
            const int c = i / G, g = i % G;
            store_coef(&qs[i], __half2float(p.q[(static_cast<int64_t>(hq) * G + g) * p.q_stride + c]));
        }
    }
    const int* kacc = p.k.acc + h * p.k.acc_hs;
    const int* vacc = p.v.acc + h * p.v.acc_hs;
    if (!is_window) {
        for (int i = tid; i <= nb; i += kThreads) {
            if (MODE != MODE_VALUE) kblk[i] = kacc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
            if (MODE != MODE_KEY) vblk[i] = vacc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
        }
    }
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const __half* knz = (MODE != MODE_VALUE) ? p.k.nz + (p.k.nz_off ? 8ll * p.k.nz_off[h] : h * p.k.nz_hs) : nullptr;
    const __half* vnz = (MODE != MODE_KEY) ? p.v.nz + (p.v.nz_off ? 8ll * p.v.nz_off[h] : h * p.v.nz_hs) : nullptr;
    const size_t stg = stage_bytes(p.cap, MODE);
    const unsigned capb = static_cast<unsigned>(p.cap) * 2u;

    // producer: bring block i of this split into stage i % kStages (thread 0 only)
    auto issue = [&](int i) {
        unsigned char* st = smem + lay.stages + static_cast<size_t>(i % kStages) * stg;
        unsigned long long* bar = &bars[i % kStages];
        const int64_t tile0 = static_cast<int64_t>(blk0 + i) * kTilesPerBlock;
        unsigned kbytes = 0, vbytes = 0, tx = 0;
        bool bad = false;
        if (MODE != MODE_VALUE) {
            const long long d = (static_cast<long long>(kblk[i + 1]) - kblk[i]) * 4;
            bad |= d < 0 || d > capb || kblk[i] < 0;
            kbytes = static_cast<unsigned>(d < 0 ? 0 : (d > capb ? capb : d)) & ~15u;
            tx += 1024 + kbytes;
        }
        if (MODE != MODE_KEY) {
            const long long d = (static_cast<long long>(vblk[i + 1]) - vblk[i]) * 4;
            bad |= d < 0 || d > capb || vblk[i] < 0;
            vbytes = static_cast<unsigned>(d < 0 ? 0 : (d > capb ? capb : d)) & ~15u;
            tx += 1024 + vbytes;
        }
        if (bad) {
            if (p.dev_status) atomicOr(p.dev_status, MFAR_DEV_BADMETA);
            kbytes = vbytes = 0;
            tx = (MODE == MODE_ATTN) ? 2048 : 1024;   // the bitmaps are still copied
        }
        mbar_expect_tx(bar, tx);
        if (MODE != MODE_VALUE) {
            bulk_g2s(st + lay.s_kbm, p.k.bmp + h * p.k.bmp_hs + tile0, 1024, bar);
            if (kbytes) bulk_g2s(st + lay.s_kval, knz + 2ll * kblk[i], kbytes, bar);
        }
        if (MODE != MODE_KEY) {
            bulk_g2s(st + lay.s_vbm, p.v.bmp + h * p.v.bmp_hs + tile0, 1024, bar);
            if (vbytes) bulk_g2s(st + lay.s_vval, vnz + 2ll * vblk[i], vbytes, bar);
        }
    };

    // per-tile offsets of the next block travel through registers (one K and one V tile per thread)
    int nxt_k = 0, nxt_v = 0;
    auto fetch_offsets = [&](int i) {
        const int64_t t = static_cast<int64_t>(blk0 + i) * kTilesPerBlock + tid;
        if (MODE != MODE_VALUE) nxt_k = kacc[t];
        if (MODE != MODE_KEY) nxt_v = vacc[t];
    };
    auto store_offsets = [&](int i) {
        const unsigned lim = static_cast<unsigned>(p.cap);
        if (MODE != MODE_VALUE) koff[(i & 1) * 128 + tid] = min(static_cast<unsigned>(2 * (nxt_k - kblk[i])), lim);
        if (MODE != MODE_KEY) voff[(i & 1) * 128 + tid] = min(static_cast<unsigned>(2 * (nxt_v - vblk[i])), lim);
    };

    if (!is_window && nb > 0) {
        if (tid == 0)
            for (int i = 0; i < min(nb, kStages - 1); ++i) issue(i);
        fetch_offsets(0);
        store_offsets(0);
    }
    __syncthreads();

    // running state
    float acc_o[8][G];   // V phase: channels 64*(gi&1) + 8*kb + i, summed over this lane's tokens
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int g = 0; g < G; ++g) acc_o[i][g] = 0.f;
    // softmax state of head g lives in warp (g % kWarps): m uniform, l a per-lane partial sum
    constexpr int kHeadsPerWarp = (G + kWarps - 1) / kWarps;
    float m_run[kHeadsPerWarp], l_run[kHeadsPerWarp];
#pragma unroll
    for (int j = 0; j < kHeadsPerWarp; ++j) { m_run[j] = -INFINITY; l_run[j] = 0.f; }

    bool timed_out = false;
    for (int i = 0; i < nb; ++i) {
        const unsigned char* st = smem + lay.stages + static_cast<size_t>(i % kStages) * stg;
        const uint2* kbm = reinterpret_cast<const uint2*>(st + lay.s_kbm);
        const uint2* vbm = reinterpret_cast<const uint2*>(st + lay.s_vbm);
        const unsigned short* kval = reinterpret_cast<const unsigned short*>(st + lay.s_kval);
        const unsigned short* vval = reinterpret_cast<const unsigned short*>(st + lay.s_vval);
        const unsigned* ko = koff + (i & 1) * 128;
        const unsigned* vo = voff + (i & 1) * 128;

        if (!is_window) {
#ifdef MFAR_ABL_NOLOAD
            if (i < kStages && !mbar_wait(&bars[i % kStages], 0)) timed_out = true;
#else
            if (i + 1 < nb) fetch_offsets(i + 1);
            if (!mbar_wait(&bars[i % kStages], (i / kStages) & 1)) timed_out = true;
#endif
        }
#ifdef MFAR_ABL_NOSYNC
        if (timed_out) break;
#else
        if (__syncthreads_or(timed_out)) { timed_out = true; break; }   // also publishes the stage hand-off below
#endif
        // every warp is done with block i-1, so its stage (untouched so far when i == 0) can
        // take block i + kStages - 1
#ifdef MFAR_ABL_NOLOAD
        if (!is_window && tid == 0 && i == 0 && kStages - 1 < nb) issue(kStages - 1);
#else
        if (!is_window && tid == 0 && i + kStages - 1 < nb) issue(i + kStages - 1);
#endif

        // ------------------------------------------------------------ K phase
        if (MODE != MODE_VALUE) {
            float acc_s[8][G];
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int g = 0; g < G; ++g) acc_s[t][g] = 0.f;
            if (!is_window) {
MFAR_UNROLL(MFAR_STEP_UNROLL)
                for (int s = 0; s < 32 / 4; ++s) {
                    const int c = warp * 32 + s * 4 + gi;
                    const uint2 bm = kbm[c];
                    coef_t coef[G];
                    load_coef<G>(qs + c * G, coef);
                    tile_step<G>(bm.y, bm.x, kval + ko[c], sel, mh, ml, coef, acc_s);
                }
            } else {
                // dense window: lane owns tokens 8*kb..8*kb+7 of this 64-token chunk, group gi
                // takes channels warp*32 + 8*gi .. +7 of each
                const int c0 = warp * 32 + gi * 8;
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const int tok = i * 64 + kb * 8 + t;
                    if (tok < W) {
                        const uint4 raw = ldg_nc_u4(p.kwin + h * p.win_hs + tok * p.win_ts + c0);
                        const __half2* hv = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __half22float2(hv[e]);
#pragma unroll
                            for (int g = 0; g < G; ++g) {
                                acc_s[t][g] = fmaf(f.x, coef_to_float(qs[(c0 + 2 * e) * G + g]), acc_s[t][g]);
                                acc_s[t][g] = fmaf(f.y, coef_to_float(qs[(c0 + 2 * e + 1) * G + g]), acc_s[t][g]);
                            }
                        }
                    }
                }
            }
            // fold lane groups (same tokens, other channels) by shuffles first when planes are to be saved
            if (kPlaneFold >= 1) {
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int g = 0; g < G; ++g) acc_s[t][g] += __shfl_xor_sync(kFull, acc_s[t][g], 16);
            }
            if (kPlaneFold >= 2) {
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int g = 0; g < G; ++g) acc_s[t][g] += __shfl_xor_sync(kFull, acc_s[t][g], 8);
            }
            // each (warp, remaining group) owns a partial plane: spart[plane][g][8*kb .. 8*kb+7]
            if (gi < kGroupsPerWarp) {
                float* dst = spart + (static_cast<size_t>(warp * kGroupsPerWarp + gi) * G) * 64 + kb * 8;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    *reinterpret_cast<float4*>(dst + g * 64) = make_float4(acc_s[0][g], acc_s[1][g], acc_s[2][g], acc_s[3][g]);
                    *reinterpret_cast<float4*>(dst + g * 64 + 4) = make_float4(acc_s[4][g], acc_s[5][g], acc_s[6][g], acc_s[7][g]);
                }
            }
        }
        if (MODE != MODE_VALUE) MFAR_LOOP_SYNC();

        // ------------------------------------------------------------ scores -> probabilities
#ifdef MFAR_ABL_NOSOFTMAX
        if (false) {
#else
        if (MODE == MODE_VALUE) {
#endif
            // p comes from the caller: warp j loads heads j, j+4, ...; lane takes tokens 2*lane, 2*lane+1
            for (int g = warp; g < G; g += kWarps) {
                const __half2 pv = *reinterpret_cast<const __half2*>(
                    p.p_in + (static_cast<int64_t>(hq) * G + g) * p.p_stride + static_cast<int64_t>(blk0 + i) * 64 + 2 * lane);
                store_coef(&ps[(2 * lane) * G + g], __low2float(pv));
                store_coef(&ps[(2 * lane + 1) * G + g], __high2float(pv));
            }
#ifdef MFAR_ABL_NOSOFTMAX
        } else if (false) {
#else
        } else {
#endif
#pragma unroll
            for (int j = 0; j < kHeadsPerWarp; ++j) {
                const int g = warp + j * kWarps;
                if (g < G) {
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int pl = 0; pl < kPlanes; ++pl) {
                        const float2 t = *reinterpret_cast<const float2*>(spart + (static_cast<size_t>(pl) * G + g) * 64 + 2 * lane);
                        s0 += t.x;
                        s1 += t.y;
                    }
                    if (MODE == MODE_KEY) {
                        *reinterpret_cast<__half2*>(p.s_out + (static_cast<int64_t>(hq) * G + g) * p.s_stride +
                                                    static_cast<int64_t>(blk0 + i) * 64 + 2 * lane) = __floats2half2_rn(s0, s1);
                    } else {
                        s0 *= p.scale_log2;
                        s1 *= p.scale_log2;
                        if (is_window) {
                            if (i * 64 + 2 * lane >= W) s0 = -INFINITY;
                            if (i * 64 + 2 * lane + 1 >= W) s1 = -INFINITY;
                        }
                        const float m_new = fmaxf(m_run[j], warp_max_f32(fmaxf(s0, s1)));
                        const float a = fast_exp2(m_run[j] - m_new);   // exp2(-inf) = 0 on the first block
                        const float p0 = round_like(ps, fast_exp2(s0 - m_new)), p1 = round_like(ps, fast_exp2(s1 - m_new));
                        l_run[j] = l_run[j] * a + (p0 + p1);
                        m_run[j] = m_new;
                        store_coef(&ps[(2 * lane) * G + g], p0);
                        store_coef(&ps[(2 * lane + 1) * G + g], p1);
                        if (lane == 0) alpha_s[g] = a;
                    }
                }
            }
        }
        if (MODE != MODE_KEY) {
#ifndef MFAR_ABL_NOLOAD
            if (!is_window && i + 1 < nb) store_offsets(i + 1);
#else
            if (!is_window && i + 1 < kStages) store_offsets(i + 1);
#endif
            MFAR_LOOP_SYNC();
        } else {
            if (i + 1 < nb) store_offsets(i + 1);
        }

        // ------------------------------------------------------------ V phase
        if (MODE != MODE_KEY) {
            if (MODE == MODE_ATTN) {
                float a[G];
                bool any = false;
#pragma unroll
                for (int g = 0; g < G; ++g) { a[g] = alpha_s[g]; any |= (a[g] != 1.f); }
                if (any) {
#pragma unroll
                    for (int t = 0; t < 8; ++t)
#pragma unroll
                        for (int g = 0; g < G; ++g) acc_o[t][g] *= a[g];
                }
            }
            const int half_id = gi & 1, par = gi >> 1;
            if (!is_window) {
MFAR_UNROLL(MFAR_STEP_UNROLL)
                for (int s = 0; s < 16 / 2; ++s) {
                    const int t = warp * 16 + s * 2 + par;
                    const int tile = half_id * 64 + t;
                    const uint2 bm = vbm[tile];
                    coef_t coef[G];
                    load_coef<G>(ps + t * G, coef);
                    tile_step<G>(bm.y, bm.x, vval + vo[tile], sel, mh, ml, coef, acc_o);
                }
            } else {
                for (int s = 0; s < 16 / 2; ++s) {
                    const int t = warp * 16 + s * 2 + par;
                    const int tok = i * 64 + t;
                    if (tok < W) {
                        const uint4 raw = ldg_nc_u4(p.vwin + h * p.win_hs + tok * p.win_ts + half_id * 64 + kb * 8);
                        const __half2* hv = reinterpret_cast<const __half2*>(&raw);
                        coef_t craw[G];
                        load_coef<G>(ps + t * G, craw);
                        float coef[G];
#pragma unroll
                        for (int g = 0; g < G; ++g) coef[g] = coef_to_float(craw[g]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __half22float2(hv[e]);
#pragma unroll
                            for (int g = 0; g < G; ++g) {
                                acc_o[2 * e][g] = fmaf(f.x, coef[g], acc_o[2 * e][g]);
                                acc_o[2 * e + 1][g] = fmaf(f.y, coef[g], acc_o[2 * e + 1][g]);
                            }
                        }
                    }
                }
            }
        }
    }

    if (timed_out) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_TIMEOUT);
        return;
    }
    if (MODE == MODE_KEY) return;

    // ---- epilogue: join token parities (lanes 16 apart), then the 4 warps, and write the partial
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
    const int nrec = (MODE == MODE_ATTN) ? p.nsplit + (p.W > 0 ? 1 : 0) : p.nsplit;
    float* rec = p.ws + ((static_cast<int64_t>(hq) * nrec + split) * G) * kPartialStride;
    for (int idx = tid; idx < G * kD; idx += kThreads) {
        const int g = idx / kD, c = idx % kD;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) s += red[(static_cast<size_t>(w) * G + g) * kD + c];
        rec[g * kPartialStride + c] = s;
    }
    if (MODE == MODE_ATTN) {
#pragma unroll
        for (int j = 0; j < kHeadsPerWarp; ++j) {
            const int g = warp + j * kWarps;
            if (g < G) {
                const float l = warp_sum_f32(l_run[j]);
                if (lane == 0) {
                    rec[g * kPartialStride + kPartM] = m_run[j];
                    rec[g * kPartialStride + kPartL] = l;
                }
            }
        }
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
template <int G, int MODE, bool MIXED>
static int launch_decode(const DecodeParams& p, int n_kv_heads, int grid_x, cudaStream_t s) {
    const SmemLayout<G, MODE> lay(p.cap);
    // largest dynamic shared memory size opted into so far, per device (and per instantiation)
    static size_t configured[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MFAR_ERR_LAUNCH;
    if (lay.total > configured[dev]) {
        if (cudaFuncSetAttribute(decode_kernel<G, MODE, MIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(lay.total)) != cudaSuccess)
            return MFAR_ERR_LAUNCH;
        configured[dev] = lay.total;
    }
    decode_kernel<G, MODE, MIXED><<<dim3(grid_x, n_kv_heads), kThreads, lay.total, s>>>(p);
    return launch_status();
}

// fp32_coef: keep q / the probabilities in fp32 (ATTN only; KEY and VALUE take fp16 coefficients as
// inputs, so the fp16 path is exact for them and always used)
template <int MODE>
static int dispatch_decode(const DecodeParams& p, int G, int n_kv_heads, int grid_x, cudaStream_t s, bool fp32_coef = false,
                           bool split8 = true) {
#define MFAR_BLK(GG)                                                                      \
    case GG:                                                                              \
        if (MODE == MODE_ATTN && fp32_coef) return launch_decode<GG, MODE, false>(p, n_kv_heads, grid_x, s); \
        return launch_decode<GG, MODE, true>(p, n_kv_heads, grid_x, s);
    switch (G) {
        MFAR_BLK(1)
        MFAR_BLK(2)
        MFAR_BLK(4)
        case 8: {
            if (!split8) {   // records in the [kv head][record][8] layout that the stream / superblock kernels write
                if (MODE == MODE_ATTN && fp32_coef) return launch_decode<8, MODE, false>(p, n_kv_heads, grid_x, s);
                return launch_decode<8, MODE, true>(p, n_kv_heads, grid_x, s);
            }
            // 8 query heads per kv head need 64 accumulators per phase and spill badly (measured 8x the time of
            // group 4); two CTAs of 4 query heads each read the same kv head instead (the second read hits L2); their partial
            // records lie in the [kv head * 2 + half][record][4] layout, which the combine kernel reads with G = 4
            DecodeParams p2 = p;
            p2.kv_share = 2 * (p.kv_share > 0 ? p.kv_share : 1);
            if (MODE == MODE_ATTN && fp32_coef) return launch_decode<4, MODE, false>(p2, 2 * n_kv_heads, grid_x, s);
            return launch_decode<4, MODE, true>(p2, 2 * n_kv_heads, grid_x, s);
        }
        default: return MFAR_ERR_ARG;
    }
#undef MFAR_BLK
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

int launch_window_record(const void* q, int64_t q_stride, int n_kv_heads, int G, const void* kwin, const void* vwin,
                         int64_t win_hs, int64_t win_ts, int W, const int* W_dev, float softmax_scale, float* ws,
                         int rec_index, unsigned* dev_status, cudaStream_t s, bool halves8) {
    if (!kwin || !vwin) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(kwin) & 15) || (reinterpret_cast<uintptr_t>(vwin) & 15) || (win_hs & 7) || (win_ts & 7))
        return MFAR_ERR_ALIGN;
    DecodeParams p{};
    p.q = static_cast<const __half*>(q);
    p.q_stride = q_stride;
    p.kwin = static_cast<const __half*>(kwin);
    p.vwin = static_cast<const __half*>(vwin);
    p.win_hs = win_hs;
    p.win_ts = win_ts;
    p.W = W;
    p.W_dev = W_dev;
    p.nsplit = rec_index;
    p.split_offset = rec_index;
    p.cap = 8;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.ws = ws;
    p.dev_status = dev_status;
    return dispatch_decode<MODE_ATTN>(p, G, n_kv_heads, 1, s, false, halves8);
}

}  // namespace mfar

using namespace mfar;

// superblock path: splits in units of 4 blocks, ~8 CTAs per SM over the whole grid
static void sb_split(int n_kv_heads, int nblk, int hint, int* ns_out, int* sps_out) {
    const int nsb = (nblk + 3) / 4;
    int ns = hint > 0 ? hint : (148 * 8 + n_kv_heads - 1) / n_kv_heads;
    if (ns > nsb) ns = nsb;
    if (ns < 1) ns = 1;
    int sps = (nsb + ns - 1) / ns;
    if (sps * 4 > 1024) sps = 256;
    *sps_out = sps;
    *ns_out = (nsb + sps - 1) / sps;
}

// Split count of the block kernel: the fitted cost model of decode_common.cuh, within the staging limit.
static int block_split(int n_kv_heads, int nblk, int hint) {
    if (nblk <= 0) return 0;
    const int min_ns = (nblk + kMaxBlocksPerSplit - 1) / kMaxBlocksPerSplit;
    int ns = hint > 0 ? hint : model_split_count(n_kv_heads, nblk, min_ns, 128);
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
    int ns_sb = 0, sps = 0;
    if (nblk > 0) sb_split(n_kv_heads, nblk, nsplit_hint, &ns_sb, &sps);
    const int recs = (ns > ns_sb ? ns : ns_sb) + 1;
    if (nsplit_out) *nsplit_out = ns;
    if (workspace_bytes)
        *workspace_bytes = static_cast<size_t>(n_kv_heads) * recs * group * kPartialStride * sizeof(float) + 16;
    return MFAR_OK;
}

static int decode_attention_fp16_impl(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, int64_t k_bmp_head_stride, const int32_t* k_accum, int64_t k_acc_head_stride,
    const void* k_nz, const int32_t* k_nz_offset, int64_t k_nz_head_stride,
    const int64_t* v_bitmaps, int64_t v_bmp_head_stride, const int32_t* v_accum, int64_t v_acc_head_stride,
    const void* v_nz, const int32_t* v_nz_offset, int64_t v_nz_head_stride,
    int n_tokens, const int32_t* n_tokens_dev, const void* k_window, const void* v_window, int64_t win_head_stride,
    int64_t win_token_stride, int window, const int32_t* window_len_dev, float softmax_scale, void* out,
    int64_t out_stride, void* workspace, size_t workspace_bytes, int nsplit, int stage_halves, int flags,
    uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens < 0 || (n_tokens % 64) || window < 0) return MFAR_ERR_ARG;
    // a device-resident length is a feature of the block kernel only
    if (n_tokens_dev && (flags & (MFAR_DECODE_FORCE_SUPERBLOCK | MFAR_DECODE_FORCE_STREAM))) return MFAR_ERR_ARG;
    if (n_tokens == 0 && window == 0) return MFAR_ERR_ARG;
    if (group != 1 && group != 2 && group != 4 && group != 8) return MFAR_ERR_ARG;
    if (!q || !out || !workspace) return MFAR_ERR_ARG;
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
                 k_nz_offset, k_bmp_head_stride, k_acc_head_stride, k_nz_head_stride};
    p.v = Sparse{reinterpret_cast<const unsigned long long*>(v_bitmaps), v_accum, static_cast<const __half*>(v_nz),
                 v_nz_offset, v_bmp_head_stride, v_acc_head_stride, v_nz_head_stride};
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
    p.ws = static_cast<float*>(workspace);
    p.dev_status = dev_status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // Two kernels: the 64-token block kernel (4 CTAs per SM) and the 256-token superblock kernel
    // (one fat CTA per SM, fewer barriers).
    const int nsb = (p.nblk + 3) / 4;
    // Measured on B200 (batch 64, 32768 tokens, group 4): block kernel 2.03 ms, superblock kernel
    // 2.55 ms, so the size heuristic currently always picks the block kernel.
    bool use_sb = false;
    (void)nsb;
    if ((flags & MFAR_DECODE_FORCE_SUPERBLOCK) && p.nblk > 0 && decode_sb_fits(p.cap, group)) use_sb = true;

    const bool use_stream = (flags & MFAR_DECODE_FORCE_STREAM) && p.nblk > 0;
    int nrec;
    int combine_group = group;
    if (use_stream) {
        const int mb = decode_stream_max_blocks();
        if (ns * mb < p.nblk) ns = (p.nblk + mb - 1) / mb;
        p.bps = (p.nblk + ns - 1) / ns;
        ns = (p.nblk + p.bps - 1) / p.bps;
        p.nsplit = ns;
        nrec = ns + (window > 0 ? 1 : 0);
        r = launch_decode_stream(p, group, n_kv_heads, (flags & MFAR_DECODE_FP16_COEF) != 0, s);
        if (r) return r;
        if (window > 0) {
            r = launch_window_record(q, q_stride, n_kv_heads, group, k_window, v_window, win_head_stride,
                                     win_token_stride, window, window_len_dev, softmax_scale, p.ws, ns, dev_status, s);
            if (r) return r;
        }
    } else if (use_sb) {
        int sps = 0;
        sb_split(n_kv_heads, p.nblk, nsplit, &ns, &sps);
        p.nsplit = ns;
        p.bps = sps;
        nrec = ns + (window > 0 ? 1 : 0);
        r = launch_decode_sb(p, group, n_kv_heads, s);
        if (r) return r;
        if (window > 0) {   // the dense window is one more record, written by the block kernel
            DecodeParams pw = p;
            pw.split_offset = ns;
            pw.cap = 8;
            r = dispatch_decode<MODE_ATTN>(pw, group, n_kv_heads, 1, s, false, false);
            if (r) return r;
        }
    } else {
        p.nsplit = ns;
        p.bps = ns > 0 ? (p.nblk + ns - 1) / ns : 0;
        nrec = ns + (window > 0 ? 1 : 0);
        r = dispatch_decode<MODE_ATTN>(p, group, n_kv_heads, nrec, s, (flags & MFAR_DECODE_FP32_COEF) != 0);
        if (r) return r;
        if (group == 8) combine_group = 4;   // the block kernel ran as two groups of 4 per kv head
    }
    combine_kernel<<<n_kv_heads * group, 128, 0, s>>>(p.ws, nrec, combine_group, 1, static_cast<__half*>(out), out_stride);
    return launch_status();
}

extern "C" int mfar_decode_attention_fp16(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, int64_t k_bmp_head_stride, const int32_t* k_accum, int64_t k_acc_head_stride,
    const void* k_nz, const int32_t* k_nz_offset, int64_t k_nz_head_stride,
    const int64_t* v_bitmaps, int64_t v_bmp_head_stride, const int32_t* v_accum, int64_t v_acc_head_stride,
    const void* v_nz, const int32_t* v_nz_offset, int64_t v_nz_head_stride,
    int n_tokens, const void* k_window, const void* v_window, int64_t win_head_stride, int64_t win_token_stride,
    int window, const int32_t* window_len_dev, float softmax_scale, void* out, int64_t out_stride, void* workspace,
    size_t workspace_bytes, int nsplit, int stage_halves, int flags, uint32_t* dev_status, void* stream) {
    return decode_attention_fp16_impl(q, q_stride, n_kv_heads, group, k_bitmaps, k_bmp_head_stride, k_accum,
                                      k_acc_head_stride, k_nz, k_nz_offset, k_nz_head_stride, v_bitmaps, v_bmp_head_stride,
                                      v_accum, v_acc_head_stride, v_nz, v_nz_offset, v_nz_head_stride, n_tokens, nullptr,
                                      k_window, v_window, win_head_stride, win_token_stride, window, window_len_dev,
                                      softmax_scale, out, out_stride, workspace, workspace_bytes, nsplit, stage_halves,
                                      flags, dev_status, stream);
}

extern "C" int mfar_decode_attention_fp16_dyn(
    const void* q, int64_t q_stride, int n_kv_heads, int group,
    const int64_t* k_bitmaps, int64_t k_bmp_head_stride, const int32_t* k_accum, int64_t k_acc_head_stride,
    const void* k_nz, const int32_t* k_nz_offset, int64_t k_nz_head_stride,
    const int64_t* v_bitmaps, int64_t v_bmp_head_stride, const int32_t* v_accum, int64_t v_acc_head_stride,
    const void* v_nz, const int32_t* v_nz_offset, int64_t v_nz_head_stride,
    int max_tokens, const int32_t* n_tokens_dev, const void* k_window, const void* v_window, int64_t win_head_stride,
    int64_t win_token_stride, int window, const int32_t* window_len_dev, float softmax_scale, void* out,
    int64_t out_stride, void* workspace, size_t workspace_bytes, int nsplit, int stage_halves, int flags,
    uint32_t* dev_status, void* stream) {
    if (!n_tokens_dev) return MFAR_ERR_ARG;
    return decode_attention_fp16_impl(q, q_stride, n_kv_heads, group, k_bitmaps, k_bmp_head_stride, k_accum,
                                      k_acc_head_stride, k_nz, k_nz_offset, k_nz_head_stride, v_bitmaps, v_bmp_head_stride,
                                      v_accum, v_acc_head_stride, v_nz, v_nz_offset, v_nz_head_stride, max_tokens,
                                      n_tokens_dev, k_window, v_window, win_head_stride, win_token_stride, window,
                                      window_len_dev, softmax_scale, out, out_stride, workspace, workspace_bytes, nsplit,
                                      stage_halves, flags, dev_status, stream);
}

extern "C" int mfar_key_scores_fp16(const void* q, int64_t q_stride, int n_kv_heads, int group,
                                    const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* accum,
                                    int64_t acc_head_stride, const void* nz, const int32_t* nz_offset,
                                    int64_t nz_head_stride, int n_tokens, void* scores, int64_t scores_stride,
                                    int stage_halves, uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens < 0 || (n_tokens % 64)) return MFAR_ERR_ARG;
    if (n_tokens == 0) return MFAR_OK;
    if (!q || !scores) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(scores) & 3) || (scores_stride & 1)) return MFAR_ERR_ALIGN;
    int r = check_sparse(bitmaps, accum, nz, bmp_head_stride, nz_head_stride);
    if (r) return r;
    DecodeParams p{};
    p.k = Sparse{reinterpret_cast<const unsigned long long*>(bitmaps), accum, static_cast<const __half*>(nz), nz_offset,
                 bmp_head_stride, acc_head_stride, nz_head_stride};
    p.q = static_cast<const __half*>(q);
    p.q_stride = q_stride;
    p.nblk = n_tokens / 64;
    // enough CTAs to fill the machine, a few blocks each so that the ring has something to overlap
    int ns = (148 * 6 + n_kv_heads - 1) / n_kv_heads;
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
    return dispatch_decode<MODE_KEY>(p, group, n_kv_heads, p.nsplit, static_cast<cudaStream_t>(stream));
}

extern "C" int mfar_value_output_fp16(const void* probs, int64_t probs_stride, int n_kv_heads, int group,
                                      const int64_t* bitmaps, int64_t bmp_head_stride, const int32_t* accum,
                                      int64_t acc_head_stride, const void* nz, const int32_t* nz_offset,
                                      int64_t nz_head_stride, int n_tokens, void* out, int64_t out_stride,
                                      void* workspace, size_t workspace_bytes, int nsplit, int stage_halves,
                                      uint32_t* dev_status, void* stream) {
    if (n_kv_heads <= 0 || group <= 0 || n_tokens <= 0 || (n_tokens % 64)) return MFAR_ERR_ARG;
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
                 bmp_head_stride, acc_head_stride, nz_head_stride};
    p.nblk = n_tokens / 64;
    p.nsplit = ns;
    p.bps = (p.nblk + ns - 1) / ns;
    p.cap = pick_cap(stage_halves);
    p.p_in = static_cast<const __half*>(probs);
    p.p_stride = probs_stride;
    p.ws = static_cast<float*>(workspace);
    p.dev_status = dev_status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    r = dispatch_decode<MODE_VALUE>(p, group, n_kv_heads, ns, s);
    const int combine_group = group == 8 ? 4 : group;
    if (r) return r;
    combine_kernel<<<n_kv_heads * group, 128, 0, s>>>(p.ws, ns, combine_group, 0, static_cast<__half*>(out), out_stride);
    return launch_status();
}
