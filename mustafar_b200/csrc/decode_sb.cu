// Fused decode attention, 256-token "superblock" variant (the fast path for long caches).
//
// One CTA per SM slot (8 or 16 warps) walks a range of superblocks = 4 consecutive
// 64-token blocks of ONE kv head, serving all G query heads of the group.
//   * staging: a 2-stage ring, each stage = 4 block slots (bitmaps + packed values of K
//     and V), filled by 1-D bulk copies (cp.async.bulk + mbarrier) one superblock ahead;
//   * K phase: lane group gi (8 lanes) works on block slot gi, lane kb on the byte
//     (8 tokens) kb of the tile; all lanes of a warp walk the same channels, each warp
//     its own slice of the 128 channels -> one partial plane of scores per warp;
//   * softmax: one warp per (query head, block slot).  Every block slot keeps its own
//     running max / sum, so no reduction across warps is needed per superblock;
//   * V phase: a warp works on tokens of one block slot only and carries output
//     accumulators relative to that slot's running max; the slots are merged once,
//     at the end of the CTA, exactly like split-KV partials;
//   * fp32 accumulation throughout.
// 3 CTA barriers per 256 tokens.  Tensor cores are not used.
#include "decode_common.cuh"

namespace mfar {

constexpr int kSbStages = 2;
constexpr int kSbMaxBlocks = 1024;   // blocks per split the offset tables can hold

typedef unsigned long long u64;

__host__ __device__ inline size_t sb_slot_bytes(int cap) { return 2048 + 2 * (static_cast<size_t>(cap) + kSlackHalves) * 2; }

template <int G, int NW>
struct SbLayout {
    size_t stages, bars, q2, spart, ps2, alpha, mstate, koff, voff, kblk, vblk, total;
    __host__ __device__ explicit SbLayout(int cap) {
        size_t o = 0;
        stages = o; o += kSbStages * 4 * sb_slot_bytes(cap);
        bars = o;   o += 64;
        q2 = o;     o += kD * G * 4;                          // [128][G]
        spart = o;  o += static_cast<size_t>(NW) * G * 256 * 4; // [warp][G][256]; reused by the epilogue
        ps2 = o;    o += 4 * 64 * G * 4;                      // [slot][64][G]
        alpha = o;  o += 4 * G * 4 + 64;                      // [slot][G]
        mstate = o; o += 2 * 4 * G * 4 + 64;                  // [slot][G] m, then [slot][G] l
        koff = o;   o += 2 * 512 * 4;
        voff = o;   o += 2 * 512 * 4;
        kblk = o;   o += (kSbMaxBlocks + 8) * 4;
        vblk = o;   o += (kSbMaxBlocks + 8) * 4;
        total = o;
    }
};

template <int G, int NW>
__global__ void __launch_bounds__(NW * 32, 1) decode_sb_kernel(DecodeParams p) {
    constexpr int kThreadsSb = NW * 32;
    constexpr int CW = kD / NW;              // channels per warp in the K phase
    constexpr int WPS = NW / 4;              // warps per block slot in the V phase
    constexpr int TW = 64 / WPS;             // tokens per warp in the V phase
    constexpr int NJ = (4 * G + NW - 1) / NW;  // (head, slot) softmax streams per warp

    extern __shared__ __align__(128) unsigned char smem[];
    const SbLayout<G, NW> lay(p.cap);
    u64* bars = reinterpret_cast<u64*>(smem + lay.bars);
    float* q2 = reinterpret_cast<float*>(smem + lay.q2);
    float* spart = reinterpret_cast<float*>(smem + lay.spart);
    float* ps2 = reinterpret_cast<float*>(smem + lay.ps2);
    float* alpha_s = reinterpret_cast<float*>(smem + lay.alpha);
    float* mstate = reinterpret_cast<float*>(smem + lay.mstate);
    unsigned* koff = reinterpret_cast<unsigned*>(smem + lay.koff);
    unsigned* voff = reinterpret_cast<unsigned*>(smem + lay.voff);
    int* kblk = reinterpret_cast<int*>(smem + lay.kblk);
    int* vblk = reinterpret_cast<int*>(smem + lay.vblk);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.y, split = blockIdx.x;
    const int gi = lane >> 3, kb = lane & 7;
    unsigned sel, mh, ml;
    lane_byte_constants(kb, sel, mh, ml);

    const int blk0 = split * p.bps * 4;                       // p.bps = superblocks per split
    const int nblocks = max(0, min(p.bps * 4, p.nblk - blk0)); // 64-token blocks of this split
    const int nsb = (nblocks + 3) / 4;

    for (int i = tid; i < kD * G; i += kThreadsSb) {
        const int c = i / G, g = i % G;
        q2[i] = __half2float(p.q[(static_cast<int64_t>(h) * G + g) * p.q_stride + c]);
    }
    const int* kacc = p.k.acc + h * p.k.acc_hs;
    const int* vacc = p.v.acc + h * p.v.acc_hs;
    for (int i = tid; i <= nblocks; i += kThreadsSb) {
        kblk[i] = kacc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
        vblk[i] = vacc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
    }
    if (tid == 0) {
        for (int s = 0; s < kSbStages; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const __half* knz = p.k.nz + (p.k.nz_off ? 8ll * p.k.nz_off[h] : h * p.k.nz_hs);
    const __half* vnz = p.v.nz + (p.v.nz_off ? 8ll * p.v.nz_off[h] : h * p.v.nz_hs);
    const size_t slotb = sb_slot_bytes(p.cap);
    const size_t val2 = (static_cast<size_t>(p.cap) + kSlackHalves) * 2;   // bytes of one value region
    const unsigned capb = static_cast<unsigned>(p.cap) * 2u;

    // producer (thread 0): superblock i -> stage i % 2
    auto issue = [&](int i) {
        unsigned char* st = smem + lay.stages + static_cast<size_t>(i % kSbStages) * 4 * slotb;
        u64* bar = &bars[i % kSbStages];
        const int nslots = min(4, nblocks - 4 * i);
        unsigned kby[4], vby[4], tx = 0;
        bool bad = false;
        for (int s = 0; s < nslots; ++s) {
            const int b = 4 * i + s;
            const long long dk = (static_cast<long long>(kblk[b + 1]) - kblk[b]) * 4;
            const long long dv = (static_cast<long long>(vblk[b + 1]) - vblk[b]) * 4;
            bad |= dk < 0 || dk > capb || dv < 0 || dv > capb || kblk[b] < 0 || vblk[b] < 0;
            kby[s] = static_cast<unsigned>(dk < 0 ? 0 : (dk > capb ? capb : dk)) & ~15u;
            vby[s] = static_cast<unsigned>(dv < 0 ? 0 : (dv > capb ? capb : dv)) & ~15u;
        }
        if (bad) {
            if (p.dev_status) atomicOr(p.dev_status, MFAR_DEV_BADMETA);
            for (int s = 0; s < nslots; ++s) kby[s] = vby[s] = 0;
        }
        for (int s = 0; s < nslots; ++s) tx += 2048 + kby[s] + vby[s];
        mbar_expect_tx(bar, tx);
        for (int s = 0; s < nslots; ++s) {
            const int b = 4 * i + s;
            unsigned char* sl = st + s * slotb;
            const int64_t tile0 = static_cast<int64_t>(blk0 + b) * kTilesPerBlock;
            bulk_g2s(sl, p.k.bmp + h * p.k.bmp_hs + tile0, 1024, bar);
            bulk_g2s(sl + 1024, p.v.bmp + h * p.v.bmp_hs + tile0, 1024, bar);
            if (kby[s]) bulk_g2s(sl + 2048, knz + 2ll * kblk[b], kby[s], bar);
            if (vby[s]) bulk_g2s(sl + 2048 + val2, vnz + 2ll * vblk[b], vby[s], bar);
        }
    };

    // per-tile offsets of the next superblock travel through registers:
    // thread t -> slot t / 128, tile t % 128 (one K and one V tile; 2 of each when NW == 8)
    constexpr int OPT = 512 / kThreadsSb;
    int nxt_k[OPT], nxt_v[OPT];
    auto fetch_offsets = [&](int i) {
#pragma unroll
        for (int r = 0; r < OPT; ++r) {
            const int e = tid + r * kThreadsSb;
            const int b = 4 * i + (e >> 7);
            if (b < nblocks) {
                const int64_t t = static_cast<int64_t>(blk0 + b) * kTilesPerBlock + (e & 127);
                nxt_k[r] = kacc[t];
                nxt_v[r] = vacc[t];
            }
        }
    };
    auto store_offsets = [&](int i) {
        const unsigned lim = static_cast<unsigned>(p.cap);
#pragma unroll
        for (int r = 0; r < OPT; ++r) {
            const int e = tid + r * kThreadsSb;
            const int b = 4 * i + (e >> 7);
            if (b < nblocks) {
                koff[(i & 1) * 512 + e] = min(static_cast<unsigned>(2 * (nxt_k[r] - kblk[b])), lim);
                voff[(i & 1) * 512 + e] = min(static_cast<unsigned>(2 * (nxt_v[r] - vblk[b])), lim);
            }
        }
    };

    if (nsb > 0) {
        if (tid == 0) issue(0);
        fetch_offsets(0);
        store_offsets(0);
    }
    __syncthreads();

    float acc_o[8][G];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int g = 0; g < G; ++g) acc_o[j][g] = 0.f;
    float m_run[NJ], l_run[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) { m_run[j] = -INFINITY; l_run[j] = 0.f; }

    bool timed_out = false;
    for (int i = 0; i < nsb; ++i) {
        const unsigned char* st = smem + lay.stages + static_cast<size_t>(i % kSbStages) * 4 * slotb;
        const unsigned* ko = koff + (i & 1) * 512;
        const unsigned* vo = voff + (i & 1) * 512;
        const int nslots = min(4, nblocks - 4 * i);

        if (i + 1 < nsb) fetch_offsets(i + 1);
        if (!mbar_wait(&bars[i % kSbStages], (i / kSbStages) & 1)) timed_out = true;
        if (__syncthreads_or(timed_out)) { timed_out = true; break; }
        // everybody is done with superblock i-1: its stage takes superblock i+1
        if (tid == 0 && i + 1 < nsb) issue(i + 1);

        // ------------------------------------------------------------ K phase
        {
            float acc_s[8][G];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int g = 0; g < G; ++g) acc_s[j][g] = 0.f;
            if (gi < nslots) {
                const unsigned char* sl = st + gi * slotb;
                const uint2* kbm = reinterpret_cast<const uint2*>(sl);
                const unsigned short* kval = reinterpret_cast<const unsigned short*>(sl + 2048);
#pragma unroll 2
                for (int s = 0; s < CW; ++s) {
                    const int c = warp * CW + s;
                    const uint2 bm = kbm[c];
                    float coef[G];
                    load_coef<G>(q2 + c * G, coef);
                    tile_step<G>(bm.y, bm.x, kval + ko[gi * 128 + c], sel, mh, ml, coef, acc_s);
                }
            }
            float* dst = spart + (static_cast<size_t>(warp) * G) * 256 + gi * 64 + kb * 8;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                *reinterpret_cast<float4*>(dst + g * 256) = make_float4(acc_s[0][g], acc_s[1][g], acc_s[2][g], acc_s[3][g]);
                *reinterpret_cast<float4*>(dst + g * 256 + 4) = make_float4(acc_s[4][g], acc_s[5][g], acc_s[6][g], acc_s[7][g]);
            }
        }
        __syncthreads();

        // ------------------------------------------------------------ softmax streams (head, slot)
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int idx = warp + j * NW;
            if (idx < 4 * G) {
                const int b = idx / G, g = idx % G;
                if (b < nslots) {
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int pl = 0; pl < NW; ++pl) {
                        const float2 t = *reinterpret_cast<const float2*>(spart + (static_cast<size_t>(pl) * G + g) * 256 + b * 64 + 2 * lane);
                        s0 += t.x;
                        s1 += t.y;
                    }
                    s0 *= p.scale_log2;
                    s1 *= p.scale_log2;
                    const float m_new = fmaxf(m_run[j], warp_max_f32(fmaxf(s0, s1)));
                    const float a = fast_exp2(m_run[j] - m_new);
                    const float p0 = fast_exp2(s0 - m_new), p1 = fast_exp2(s1 - m_new);
                    l_run[j] = l_run[j] * a + (p0 + p1);
                    m_run[j] = m_new;
                    ps2[(b * 64 + 2 * lane) * G + g] = p0;
                    ps2[(b * 64 + 2 * lane + 1) * G + g] = p1;
                    if (lane == 0) alpha_s[b * G + g] = a;
                }
            }
        }
        if (i + 1 < nsb) store_offsets(i + 1);
        __syncthreads();

        // ------------------------------------------------------------ V phase
        {
            const int b = warp / WPS, sub = warp % WPS;
            if (b < nslots) {
                bool any = false;
                float a[G];
#pragma unroll
                for (int g = 0; g < G; ++g) { a[g] = alpha_s[b * G + g]; any |= (a[g] != 1.f); }
                if (any) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
#pragma unroll
                        for (int g = 0; g < G; ++g) acc_o[j][g] *= a[g];
                }
                const unsigned char* sl = st + b * slotb;
                const uint2* vbm = reinterpret_cast<const uint2*>(sl + 1024);
                const unsigned short* vval = reinterpret_cast<const unsigned short*>(sl + 2048 + val2);
                const int half_id = gi & 1, par = gi >> 1;
#pragma unroll 2
                for (int s = 0; s < TW / 2; ++s) {
                    const int t = sub * TW + s * 2 + par;
                    const int tile = half_id * 64 + t;
                    const uint2 bm = vbm[tile];
                    float coef[G];
                    load_coef<G>(ps2 + (b * 64 + t) * G, coef);
                    tile_step<G>(bm.y, bm.x, vval + vo[b * 128 + tile], sel, mh, ml, coef, acc_o);
                }
            }
        }
    }

    if (timed_out) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_TIMEOUT);
        return;
    }

    // ---- epilogue: merge the 4 block-slot streams (each has its own running max), then the warps
    __syncthreads();
    float* m_s = mstate;            // [slot][G]
    float* l_s = mstate + 4 * G;    // [slot][G]
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int idx = warp + j * NW;
        if (idx < 4 * G) {
            const float l = warp_sum_f32(l_run[j]);
            if (lane == 0) { m_s[idx] = m_run[j]; l_s[idx] = l; }   // idx = slot * G + g
        }
    }
    __syncthreads();
    {
        const int b = warp / WPS;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float M = -INFINITY;
#pragma unroll
            for (int s = 0; s < 4; ++s) M = fmaxf(M, m_s[s * G + g]);
            const float mb = m_s[b * G + g];
            const float w = (mb == -INFINITY) ? 0.f : fast_exp2(mb - M);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc_o[j][g] *= w;
        }
    }
    float* red = spart;   // [warp][G][128]
    {
        const int ch = (gi & 1) * 64 + kb * 8;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = acc_o[j][g] + __shfl_xor_sync(kFull, acc_o[j][g], 16);
            if (lane < 16) {
                float* d = red + (static_cast<size_t>(warp) * G + g) * kD + ch;
                *reinterpret_cast<float4*>(d) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(d + 4) = make_float4(f[4], f[5], f[6], f[7]);
            }
        }
    }
    __syncthreads();
    const int nrec = p.nsplit + (p.W > 0 ? 1 : 0);
    float* rec = p.ws + ((static_cast<int64_t>(h) * nrec + split) * G) * kPartialStride;
    for (int idx = tid; idx < G * kD; idx += kThreadsSb) {
        const int g = idx / kD, c = idx % kD;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) s += red[(static_cast<size_t>(w) * G + g) * kD + c];
        rec[g * kPartialStride + c] = s;
    }
    if (tid < G) {
        const int g = tid;
        float M = -INFINITY;
        for (int s = 0; s < 4; ++s) M = fmaxf(M, m_s[s * G + g]);
        float l = 0.f;
        for (int s = 0; s < 4; ++s) {
            const float ms = m_s[s * G + g];
            if (ms != -INFINITY) l += l_s[s * G + g] * fast_exp2(ms - M);
        }
        rec[g * kPartialStride + kPartM] = M;
        rec[g * kPartialStride + kPartL] = l;
    }
}

template <int G, int NW>
static int launch_sb(const DecodeParams& p, int n_kv_heads, cudaStream_t s) {
    const SbLayout<G, NW> lay(p.cap);
    static size_t configured[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MFAR_ERR_LAUNCH;
    if (lay.total > configured[dev]) {
        if (cudaFuncSetAttribute(decode_sb_kernel<G, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(lay.total)) != cudaSuccess)
            return MFAR_ERR_LAUNCH;
        configured[dev] = lay.total;
    }
    decode_sb_kernel<G, NW><<<dim3(p.nsplit, n_kv_heads), NW * 32, lay.total, s>>>(p);
    return launch_status();
}

constexpr size_t kSmemLimit = 227 * 1024;

template <int G>
static int pick_nw(int cap) {
    if (SbLayout<G, 16>(cap).total <= kSmemLimit) return 16;
    if (SbLayout<G, 8>(cap).total <= kSmemLimit) return 8;
    return 0;
}

static int sb_nw(int cap, int G) {
    switch (G) {
        case 1: return pick_nw<1>(cap);
        case 2: return pick_nw<2>(cap);
        case 4: return pick_nw<4>(cap);
        case 8: return pick_nw<8>(cap) == 16 ? 8 : pick_nw<8>(cap);   // 16 warps x 8 heads does not fit the register file
        default: return 0;
    }
}

bool decode_sb_fits(int cap, int G) { return sb_nw(cap, G) != 0; }

int launch_decode_sb(const DecodeParams& p, int G, int n_kv_heads, cudaStream_t s) {
    const int nw = sb_nw(p.cap, G);
    if (nw == 0) return MFAR_ERR_ARG;
#define MFAR_SB(GG)                                                        \
    case GG:                                                               \
        return nw == 16 ? launch_sb<GG, 16>(p, n_kv_heads, s) : launch_sb<GG, 8>(p, n_kv_heads, s);
    switch (G) {
        MFAR_SB(1)
        MFAR_SB(2)
        MFAR_SB(4)
        case 8: return launch_sb<8, 8>(p, n_kv_heads, s);
        default: return MFAR_ERR_ARG;
    }
#undef MFAR_SB
}

}  // namespace mfar
