// Fused decode attention over the bitmap + packed-fp16 cache:
//   q.K^T over the compressed tokens, online softmax, P.V, split-KV partial records, and the merge of the
//   records by the CTA that finishes a kv head last (one launch per call); one extra CTA per kv head handles
//   the dense recent-token window.
//
// A CTA (4 warps) walks a range of 64-token blocks of ONE kv head and serves all G query heads that share it, so
// the compressed bytes are read once.  Per block the two bitmap arrays (1 KiB each) and the two packed-value
// ranges travel into a 2-stage shared-memory ring by 1-D bulk copies (cp.async.bulk + mbarrier, no multicast),
// issued by one thread one block ahead.
//
// Decode: a lane owns one BYTE (8 positions) of the bitmaps of TWO tiles.  The rank of the byte's first position is
// the popcount of the bitmap bits before it; every set bit then takes the next packed half from shared memory
// (a predicated 16-bit load), absent positions stay zero, and the two tiles' values at the same position are packed
// into one 32-bit register.  Those registers ARE fragments of mma.sync.m16n8k16 (fp16 in, fp32 accumulate):
//   K phase   S[token][head]   = sum_c K[token][c] q[c][head]     rows = tokens,   k = channels (= K tiles)
//   V phase   O[channel][head] = sum_t V[t][channel] p[t][head]   rows = channels, k = tokens   (= V tiles)
// In both phases the position inside a tile is the row and the tile index is the contraction index, which is exactly
// how the A fragment spreads over a warp (row = lane / 4, k pair = lane % 4), so no transposition is needed.  The
// query heads (up to 8) are the n dimension.  The multiply-accumulate of a 64-token block is 64 tensor-core
// instructions per CTA; what remains, and what bounds the kernel, is the shared-memory traffic of the
// predicated loads.
//
// The same kernel serves the quantised cache (QBITS = 2 or 4): there a tile's code words, bitmap, scale and zero-point
// are staged by the threads themselves (4-byte cp.async, one tile of each tensor per thread, one block ahead); a lane
// takes the codes of its byte out of a 32-bit window that starts at its rank, turns every code into
// fp16((code - zero) * scale) with the subtraction and the product in fp32 - the reference's arithmetic
// (kernel_quant/csrc/SpMM_Kernel_Quant.cuh:235-240) - and packs the two tiles' values into the same fragments.
// No per-position shared-memory load is left, so that variant is bound by instruction issue.
#include "decode_common.cuh"

namespace mfar {

constexpr int kAWarps = 4;
constexpr int kAThreads = kAWarps * 32;
constexpr int kAStages = 2;
constexpr int kPsStride = 72;      // halves per probability row: 36 words, so the 8 head rows fall in different banks
constexpr int kPlaneStride = 72;   // floats per (warp, head) score plane

__host__ __device__ inline size_t attn_stage_bytes(int cap) {
    return 2 * (1024 + (static_cast<size_t>(cap) + kSlackHalves) * 2);
}

struct AttnLayout {
    size_t stages, bars, ps, red, alpha, koff, voff, kblk, vblk, total;
    size_t s_kbm, s_vbm, s_kval, s_vval;
    // qbuf_bytes > 0: quantised cache, a stage is two QBuf (K then V) instead of bitmaps + packed halves
    __host__ __device__ AttnLayout(int cap, int G, size_t qbuf_bytes = 0) {
        s_kbm = 0;
        s_vbm = 1024;
        s_kval = 2048;
        s_vval = 2048 + (static_cast<size_t>(cap) + kSlackHalves) * 2;
        size_t o = 0;
        stages = o; o += kAStages * (qbuf_bytes ? 2 * qbuf_bytes : attn_stage_bytes(cap));
        bars = o;   o += 64;
        ps = o;     o += 8 * kPsStride * 2;
        red = o;    o += static_cast<size_t>(kAWarps) * G * kD * 4;   // score planes, later the output reduction
        alpha = o;  o += 64;
        koff = o;   o += 2 * 128 * 4;
        voff = o;   o += 2 * 128 * 4;
        kblk = o;   o += (kMaxBlocksPerSplit + 4) * 4;
        vblk = o;   o += (kMaxBlocksPerSplit + 4) * 4;
        total = o;
    }
};

__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte `sel` (8 positions) of two tiles -> 8 registers, low half = tile A, high half = tile B, zero where the bit
// is clear.  bm = {lo A, hi A, lo B, hi B}; va / vb point at the tiles' packed values.
__device__ __forceinline__ void expand_pair(uint4 bm, const unsigned short* va, const unsigned short* vb, unsigned sel,
                                            unsigned mh, unsigned ml, unsigned (&r)[8]) {
    const unsigned ba = __byte_perm(bm.x, bm.y, sel), bb = __byte_perm(bm.z, bm.w, sel);
    const unsigned short* pa[2];
    const unsigned short* pb[2];
    pa[0] = va + (__popc(bm.y & mh) + __popc(bm.x & ml));
    pb[0] = vb + (__popc(bm.w & mh) + __popc(bm.z & ml));
    pa[1] = pa[0] + __popc(ba & 0xf0u);
    pb[1] = pb[0] + __popc(bb & 0xf0u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        // one zero per register: tile A's half is loaded straight into it, tile B's half is merged in only when present
        unsigned v = 0;
        if (ba & (0x80u >> i)) { v = *pa[i / 4]; ++pa[i / 4]; }
        if (bb & (0x80u >> i)) { const unsigned hi = *pb[i / 4]; ++pb[i / 4]; v = __byte_perm(v, hi, 0x5410); }
        r[i] = v;
    }
}


__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Quantised counterpart of expand_pair: byte `sel` of tiles c and c + 1 of a staged block.  A lane's codes are
// consecutive in the tile's code words from bit rank * BITS on; every set bit takes the next code.
template <int BITS, bool GROUP32>
__device__ __forceinline__ void expand_pair_q(const QBuf<BITS>& b, int c, unsigned sel, unsigned mh, unsigned ml,
                                              unsigned (&r)[8]) {
    constexpr unsigned MASK = (1u << BITS) - 1u;
    constexpr int WPT = QBuf<BITS>::WPT;
    const uint4 bm = *reinterpret_cast<const uint4*>(&b.bm[c]);
    const uint4 sz = *reinterpret_cast<const uint4*>(&b.sz[2 * c]);   // (scale | zero << 16): A group 0, 1; B group 0, 1
    const unsigned ba = __byte_perm(bm.x, bm.y, sel), bb = __byte_perm(bm.z, bm.w, sel);
    int ra = __popc(bm.y & mh) + __popc(bm.x & ml), rb = __popc(bm.w & mh) + __popc(bm.z & ml);
    const unsigned oa = static_cast<unsigned>(ra) * BITS, ob = static_cast<unsigned>(rb) * BITS;
    const unsigned* wa = b.words + c * WPT + (oa >> 5);
    const unsigned* wb = b.words + (c + 1) * WPT + (ob >> 5);
    unsigned wina = __funnelshift_r(wa[0], wa[1], oa & 31u), winb = __funnelshift_r(wb[0], wb[1], ob & 31u);
    auto scale_of = [](unsigned x) { return __half2float(__ushort_as_half(static_cast<unsigned short>(x & 0xffffu))); };
    // code - zero exactly: the code is or-ed into the mantissa of 2^23, the zero-point is offset by 2^23 as well
    auto zero_of = [](unsigned x) { return 8388608.f + __half2float(__ushort_as_half(static_cast<unsigned short>(x >> 16))); };
    const float sa0 = scale_of(sz.x), za0 = zero_of(sz.x), sb0 = scale_of(sz.z), zb0 = zero_of(sz.z);
    float sa1 = sa0, za1 = za0, sb1 = sb0, zb1 = zb0;
    if (GROUP32) { sa1 = scale_of(sz.y); za1 = zero_of(sz.y); sb1 = scale_of(sz.w); zb1 = zero_of(sz.w); }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float va = 0.f, vb = 0.f;
        if (ba & (0x80u >> i)) {
            const bool second = GROUP32 && ra >= 32;   // nonzeros 32.. of a tile use the second scale / zero-point
            va = (__uint_as_float(0x4b000000u | (wina & MASK)) - (second ? za1 : za0)) * (second ? sa1 : sa0);
            wina >>= BITS;
            if (GROUP32) ++ra;
        }
        if (bb & (0x80u >> i)) {
            const bool second = GROUP32 && rb >= 32;
            vb = (__uint_as_float(0x4b000000u | (winb & MASK)) - (second ? zb1 : zb0)) * (second ? sb1 : sb0);
            winb >>= BITS;
            if (GROUP32) ++rb;
        }
        const __half2 h2 = __floats2half2_rn(va, vb);
        r[i] = *reinterpret_cast<const unsigned*>(&h2);
    }
}

__device__ __forceinline__ unsigned ldg_nc_u32(const void* p) {
    unsigned v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned ldg_nc_u16(const void* p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ldcg_f32x4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldcg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// record of (kv head h, split, query head g) inside the workspace
__device__ __forceinline__ float* record_ptr(const DecodeParams& p, int G, int h, int split, int g) {
    const int rg = p.rec_group;
    const int sets = G / rg;
    return p.ws + ((static_cast<int64_t>(h * sets + g / rg) * p.nrec + split) * rg + (g % rg)) * kPartialStride;
}

template <int G, int QBITS, bool GROUP32>
__global__ void __launch_bounds__(kAThreads, 4) decode_attn_kernel(DecodeParams p) {
    constexpr bool QUANT = QBITS != 0;
    using QB = QBuf<QUANT ? QBITS : 2>;
    extern __shared__ __align__(128) unsigned char smem[];
    const AttnLayout lay(p.cap, G, QUANT ? sizeof(QB) : 0);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + lay.bars);
    unsigned short* ps = reinterpret_cast<unsigned short*>(smem + lay.ps);    // [8][kPsStride] probabilities, fp16
    float* red = reinterpret_cast<float*>(smem + lay.red);                     // [warp][G][kPlaneStride] scores
    float* alpha_s = reinterpret_cast<float*>(smem + lay.alpha);               // [8]
    unsigned* koff = reinterpret_cast<unsigned*>(smem + lay.koff);             // [2][128] halves, relative to the block
    unsigned* voff = reinterpret_cast<unsigned*>(smem + lay.voff);
    int* kblk = reinterpret_cast<int*>(smem + lay.kblk);                       // block starts (uint32 units) of this split
    int* vblk = reinterpret_cast<int*>(smem + lay.vblk);
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tb = lane >> 2, cp = lane & 3;   // fragment row (= bitmap byte) and k pair of this lane
    const int h = blockIdx.y;
    const int split = blockIdx.x + p.split_offset;
    const bool is_window = split == p.nsplit;
    unsigned sel, mh, ml;
    lane_byte_constants(tb, sel, mh, ml);

    // the compressed length may live in device memory (a captured launch keeps working while blocks are appended):
    // p.nblk is then its upper bound, the grid was sized for that bound, and the blocks actually there are dealt
    // out again over the same number of splits (splits past the end write an empty record)
    int nblk = p.nblk, bps = p.bps;
    if (p.L_dev) {
        nblk = max(0, min(*p.L_dev / 64, p.nblk));
        bps = p.nsplit > 0 ? (nblk + p.nsplit - 1) / p.nsplit : 0;
    }
    const int blk0 = is_window ? 0 : split * bps;
    const int W = (is_window && p.W_dev) ? max(0, min(*p.W_dev, p.W)) : p.W;
    int nb = is_window ? (W + 63) / 64 : min(bps, nblk - blk0);
    if (nb < 0) nb = 0;

    // ---- prologue
    // q fragments (B operand of the K phase) of this warp's 32 channels: n = head tb, k pairs 2*cp, 2*cp+1 (+8)
    unsigned qb[2][2] = {{0u, 0u}, {0u, 0u}};
    if (tb < G) {
        const __half* qrow = p.q + (static_cast<int64_t>(h) * G + tb) * p.q_stride + warp * 32 + 2 * cp;
#pragma unroll
        for (int kg = 0; kg < 2; ++kg)
#pragma unroll
            for (int j = 0; j < 2; ++j) qb[kg][j] = ldg_nc_u32(qrow + kg * 16 + j * 8);
    }
    for (int i = tid; i < 8 * kPsStride / 2; i += kAThreads) reinterpret_cast<unsigned*>(ps)[i] = 0u;
    const int* kacc = QUANT ? nullptr : p.k.acc + h * p.k.acc_hs;
    const int* vacc = QUANT ? nullptr : p.v.acc + h * p.v.acc_hs;
    if (!QUANT && !is_window) {
        for (int i = tid; i <= nb; i += kAThreads) {
            kblk[i] = kacc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
            vblk[i] = vacc[static_cast<int64_t>(blk0 + i) * kTilesPerBlock];
        }
    }
    if (tid == 0) {
        for (int s = 0; s < kAStages; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const int64_t k_head0 = QUANT ? 0 : (p.k.nz_off ? 8ll * p.k.nz_off[h] : h * p.k.nz_hs);
    const int64_t v_head0 = QUANT ? 0 : (p.v.nz_off ? 8ll * p.v.nz_off[h] : h * p.v.nz_hs);
    const __half* knz = p.k.nz + k_head0;
    const __half* vnz = p.v.nz + v_head0;
    const size_t stg = attn_stage_bytes(p.cap);
    const unsigned capb = static_cast<unsigned>(p.cap) * 2u;

    // producer: bring block i of this split into stage i % kAStages (thread 0 only)
    auto issue = [&](int i) {
        unsigned char* st = smem + lay.stages + static_cast<size_t>(i % kAStages) * stg;
        unsigned long long* bar = &bars[i % kAStages];
        const int64_t tile0 = static_cast<int64_t>(blk0 + i) * kTilesPerBlock;
        unsigned kbytes = static_cast<unsigned>(kblk[i + 1] - kblk[i]) * 4u;
        unsigned vbytes = static_cast<unsigned>(vblk[i + 1] - vblk[i]) * 4u;
        const bool bad = block_range_bad(kblk[i], kblk[i + 1], capb, k_head0, p.k.nz_extent) ||
                         block_range_bad(vblk[i], vblk[i + 1], capb, v_head0, p.v.nz_extent);
        if (bad) {   // the bitmaps are still copied, the values are not
            if (p.dev_status) atomicOr(p.dev_status, MFAR_DEV_BADMETA);
            kbytes = vbytes = 0;
        }
        mbar_expect_tx(bar, 2048 + kbytes + vbytes);
        bulk_g2s(st + lay.s_kbm, p.k.bmp + h * p.k.bmp_hs + tile0, 1024, bar);
        if (kbytes) bulk_g2s(st + lay.s_kval, knz + 2ll * kblk[i], kbytes, bar);
        bulk_g2s(st + lay.s_vbm, p.v.bmp + h * p.v.bmp_hs + tile0, 1024, bar);
        if (vbytes) bulk_g2s(st + lay.s_vval, vnz + 2ll * vblk[i], vbytes, bar);
    };

    // per-tile offsets of the next block travel through registers (one K and one V tile per thread)
    int nxt_k = 0, nxt_v = 0;
    auto fetch_offsets = [&](int i) {
        const int64_t t = static_cast<int64_t>(blk0 + i) * kTilesPerBlock + tid;
        nxt_k = kacc[t];
        nxt_v = vacc[t];
    };
    auto store_offsets = [&](int i) {
        const unsigned lim = static_cast<unsigned>(p.cap);
        koff[(i & 1) * 128 + tid] = min(static_cast<unsigned>(2 * (nxt_k - kblk[i])), lim);
        voff[(i & 1) * 128 + tid] = min(static_cast<unsigned>(2 * (nxt_v - vblk[i])), lim);
    };

    // quantised cache: thread t owns K tile t and V tile t of a block; their metadata travels through registers
    // one block ahead, the code words go straight to the tile's slot of the stage
    struct Meta { uint2 bm; int off; unsigned sz[2]; };
    Meta mk{}, mv{};
    auto q_load_meta = [&](const QSparse& sp, int i, Meta& m) {
        const int64_t t = static_cast<int64_t>(blk0 + i) * kTilesPerBlock + tid;
        const unsigned long long bmw = sp.bmp[h * sp.bmp_hs + t];
        m.bm = make_uint2(static_cast<unsigned>(bmw), static_cast<unsigned>(bmw >> 32));
        const int64_t mi = h * sp.meta_hs + t;
        m.off = sp.tile_off[mi];
        const int ngrp = GROUP32 ? 2 : 1;
        m.sz[1] = 0u;
        for (int g = 0; g < ngrp; ++g)
            m.sz[g] = static_cast<unsigned>(__half_as_ushort(sp.scales[mi * ngrp + g])) |
                      (static_cast<unsigned>(__half_as_ushort(sp.zeros[mi * ngrp + g])) << 16);
    };
    auto q_stage = [&](const QSparse& sp, const Meta& m, QB& b) {
        constexpr int CAPW = 32 / (QUANT ? QBITS : 2);
        b.bm[tid] = m.bm;
        b.sz[2 * tid] = m.sz[0];
        b.sz[2 * tid + 1] = m.sz[1];
        const int n = (__popc(m.bm.x) + __popc(m.bm.y) + CAPW - 1) / CAPW;
        if (m.off < 0 || static_cast<long long>(m.off) + n > sp.packed_words) {
            if (n > 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_BADMETA);
            b.bm[tid] = make_uint2(0u, 0u);     // the tile contributes nothing
            return;
        }
        const unsigned* src = sp.packed + m.off;
        for (int j = 0; j < n; ++j) cp_async4(&b.words[tid * QB::WPT + j], src + j);
    };
    auto qbuf = [&](int i, int which) -> QB& {
        return *reinterpret_cast<QB*>(smem + lay.stages + (static_cast<size_t>(i % kAStages) * 2 + which) * sizeof(QB));
    };

    if (!is_window && nb > 0) {
        if (QUANT) {
            q_load_meta(p.kq, 0, mk);
            q_load_meta(p.vq, 0, mv);
            q_stage(p.kq, mk, qbuf(0, 0));
            q_stage(p.vq, mv, qbuf(0, 1));
            cp_async_commit();
            if (nb > 1) { q_load_meta(p.kq, 1, mk); q_load_meta(p.vq, 1, mv); }
        } else {
            if (tid == 0)
                for (int i = 0; i < min(nb, kAStages - 1); ++i) issue(i);
            fetch_offsets(0);
            store_offsets(0);
        }
    }
    __syncthreads();

    // running state.  dv[hf][i]: rows = channels 64*hf + 8*tb + i (d0, d1) and + 4 (d2, d3); columns = heads 2*cp, 2*cp+1
    float dv[2][4][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) dv[a][i][e] = 0.f;
    // softmax state of head g lives in warp g % 4: m uniform, l a per-lane partial sum
    constexpr int kHeadsPerWarp = (G + kAWarps - 1) / kAWarps;
    float m_run[kHeadsPerWarp], l_run[kHeadsPerWarp];
#pragma unroll
    for (int j = 0; j < kHeadsPerWarp; ++j) { m_run[j] = -INFINITY; l_run[j] = 0.f; }

    bool timed_out = false;
    for (int i = 0; i < nb; ++i) {
        const unsigned char* st = smem + lay.stages + static_cast<size_t>(i % kAStages) * stg;
        const uint2* kbm = reinterpret_cast<const uint2*>(st + lay.s_kbm);
        const uint2* vbm = reinterpret_cast<const uint2*>(st + lay.s_vbm);
        const unsigned short* kval = reinterpret_cast<const unsigned short*>(st + lay.s_kval);
        const unsigned short* vval = reinterpret_cast<const unsigned short*>(st + lay.s_vval);
        const unsigned* ko = koff + (i & 1) * 128;
        const unsigned* vo = voff + (i & 1) * 128;

        if (!is_window) {
            if (QUANT) {
                cp_async_wait_all();
            } else {
                if (i + 1 < nb) fetch_offsets(i + 1);
                if (!mbar_wait(&bars[i % kAStages], (i / kAStages) & 1)) timed_out = true;
            }
        }
        if (__syncthreads_or(timed_out)) { timed_out = true; break; }   // also publishes the stage hand-off below
        // every warp is done with block i-1, so its stage can take block i + kAStages - 1
        if (!is_window) {
            if (QUANT) {
                if (i + 1 < nb) {
                    q_stage(p.kq, mk, qbuf(i + 1, 0));
                    q_stage(p.vq, mv, qbuf(i + 1, 1));
                    cp_async_commit();
                    if (i + 2 < nb) { q_load_meta(p.kq, i + 2, mk); q_load_meta(p.vq, i + 2, mv); }
                }
            } else if (tid == 0 && i + kAStages - 1 < nb) {
                issue(i + kAStages - 1);
            }
        }

        // ------------------------------------------------------------ K phase: this warp's 32 channels x 64 tokens
        // dk[j]: rows = tokens 8*tb + j (d0, d1) and 8*tb + j + 4 (d2, d3); columns = heads 2*cp, 2*cp+1
        float dk[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) dk[j][e] = 0.f;
        if (!is_window) {
#pragma unroll
            for (int kg = 0; kg < 2; ++kg) {
                unsigned r1[8], r2[8];
                if (QUANT) {
                    const int c = warp * 32 + kg * 16 + 2 * cp;
                    expand_pair_q<QB::BITS, GROUP32>(qbuf(i, 0), c, sel, mh, ml, r1);
                    expand_pair_q<QB::BITS, GROUP32>(qbuf(i, 0), c + 8, sel, mh, ml, r2);
                } else {
                    {
                        const int c = warp * 32 + kg * 16 + 2 * cp;
                        const uint4 bm = *reinterpret_cast<const uint4*>(kbm + c);
                        const uint2 of = *reinterpret_cast<const uint2*>(ko + c);
                        expand_pair(bm, kval + of.x, kval + of.y, sel, mh, ml, r1);
                    }
                    {
                        const int c = warp * 32 + kg * 16 + 8 + 2 * cp;
                        const uint4 bm = *reinterpret_cast<const uint4*>(kbm + c);
                        const uint2 of = *reinterpret_cast<const uint2*>(ko + c);
                        expand_pair(bm, kval + of.x, kval + of.y, sel, mh, ml, r2);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) mma16816(dk[j], r1[j], r1[j + 4], r2[j], r2[j + 4], qb[kg][0], qb[kg][1]);
            }
        } else {
            // dense window: the A fragment is two adjacent channels of one token, a 32-bit load
            const __half* kw = p.kwin + h * p.win_hs;
#pragma unroll
            for (int kg = 0; kg < 2; ++kg) {
                const int c = warp * 32 + kg * 16 + 2 * cp;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int t0 = i * 64 + 8 * tb + j, t1 = t0 + 4;
                    unsigned a0 = 0, a1 = 0, a2 = 0, a3 = 0;
                    if (t0 < W) { a0 = ldg_nc_u32(kw + t0 * p.win_ts + c); a2 = ldg_nc_u32(kw + t0 * p.win_ts + c + 8); }
                    if (t1 < W) { a1 = ldg_nc_u32(kw + t1 * p.win_ts + c); a3 = ldg_nc_u32(kw + t1 * p.win_ts + c + 8); }
                    mma16816(dk[j], a0, a1, a2, a3, qb[kg][0], qb[kg][1]);
                }
            }
        }
        // score planes [warp][head][slot], slot = 8*j + tb for token 8*tb + j (consecutive lanes, consecutive words)
        {
            float* pl = red + static_cast<size_t>(warp) * G * kPlaneStride;
            if (2 * cp < G) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    pl[(2 * cp) * kPlaneStride + j * 8 + tb] = dk[j][0];
                    pl[(2 * cp) * kPlaneStride + (j + 4) * 8 + tb] = dk[j][2];
                }
            }
            if (2 * cp + 1 < G) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    pl[(2 * cp + 1) * kPlaneStride + j * 8 + tb] = dk[j][1];
                    pl[(2 * cp + 1) * kPlaneStride + (j + 4) * 8 + tb] = dk[j][3];
                }
            }
        }
        __syncthreads();

        // ------------------------------------------------------------ scores -> probabilities (warp g % 4 owns head g)
#pragma unroll
        for (int j = 0; j < kHeadsPerWarp; ++j) {
            const int g = warp + j * kAWarps;
            if (g < G) {
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int w = 0; w < kAWarps; ++w) {
                    const float2 t = *reinterpret_cast<const float2*>(red + (static_cast<size_t>(w) * G + g) * kPlaneStride + 2 * lane);
                    s0 += t.x;
                    s1 += t.y;
                }
                // slots 2*lane, 2*lane + 1 hold tokens 16*(lane % 4) + lane / 4 and + 8
                const int tok0 = 16 * (lane & 3) + (lane >> 2), tok1 = tok0 + 8;
                s0 *= p.scale_log2;
                s1 *= p.scale_log2;
                if (is_window) {
                    if (i * 64 + tok0 >= W) s0 = -INFINITY;
                    if (i * 64 + tok1 >= W) s1 = -INFINITY;
                }
                const float m_new = fmaxf(m_run[j], warp_max_f32(fmaxf(s0, s1)));
                const float a = fast_exp2(m_run[j] - m_new);   // exp2(-inf) = 0 on the first block
                // the probability that enters P.V is rounded to fp16 (as the reference model does before its
                // value op); the running sum uses the same rounded value
                const __half h0 = __float2half_rn(fast_exp2(s0 - m_new)), h1 = __float2half_rn(fast_exp2(s1 - m_new));
                l_run[j] = l_run[j] * a + (__half2float(h0) + __half2float(h1));
                m_run[j] = m_new;
                ps[g * kPsStride + tok0] = __half_as_ushort(h0);
                ps[g * kPsStride + tok1] = __half_as_ushort(h1);
                if (lane == 0) alpha_s[g] = a;
            }
        }
        if (!QUANT && !is_window && i + 1 < nb) store_offsets(i + 1);
        __syncthreads();

        // ------------------------------------------------------------ V phase: this warp's 16 tokens x 128 channels
        {
            float a0 = 1.f, a1 = 1.f;
            if (2 * cp < G) a0 = alpha_s[2 * cp];
            if (2 * cp + 1 < G) a1 = alpha_s[2 * cp + 1];
            if (__any_sync(kFull, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        dv[hf][j][0] *= a0; dv[hf][j][1] *= a1;
                        dv[hf][j][2] *= a0; dv[hf][j][3] *= a1;
                    }
            }
        }
        // probabilities as the B operand: n = head tb, k pairs = tokens 16*warp + 2*cp, +1 (+8)
        const unsigned pb0 = *reinterpret_cast<const unsigned*>(ps + tb * kPsStride + warp * 16 + 2 * cp);
        const unsigned pb1 = *reinterpret_cast<const unsigned*>(ps + tb * kPsStride + warp * 16 + 8 + 2 * cp);
        if (!is_window) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                unsigned r1[8], r2[8];
                if (QUANT) {
                    const int t = hf * 64 + warp * 16 + 2 * cp;
                    expand_pair_q<QB::BITS, GROUP32>(qbuf(i, 1), t, sel, mh, ml, r1);
                    expand_pair_q<QB::BITS, GROUP32>(qbuf(i, 1), t + 8, sel, mh, ml, r2);
                } else {
                    {
                        const int t = hf * 64 + warp * 16 + 2 * cp;
                        const uint4 bm = *reinterpret_cast<const uint4*>(vbm + t);
                        const uint2 of = *reinterpret_cast<const uint2*>(vo + t);
                        expand_pair(bm, vval + of.x, vval + of.y, sel, mh, ml, r1);
                    }
                    {
                        const int t = hf * 64 + warp * 16 + 8 + 2 * cp;
                        const uint4 bm = *reinterpret_cast<const uint4*>(vbm + t);
                        const uint2 of = *reinterpret_cast<const uint2*>(vo + t);
                        expand_pair(bm, vval + of.x, vval + of.y, sel, mh, ml, r2);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) mma16816(dv[hf][j], r1[j], r1[j + 4], r2[j], r2[j + 4], pb0, pb1);
            }
        } else {
            // dense window: the A fragment pairs two adjacent tokens of one channel (two 16-bit loads)
            const __half* vw = p.vwin + h * p.win_hs;
            const int tA = i * 64 + warp * 16 + 2 * cp;
            auto pair = [&](int t, int ch) -> unsigned {
                unsigned lo = 0, hi = 0;
                if (t < W) lo = ldg_nc_u16(vw + t * p.win_ts + ch);
                if (t + 1 < W) hi = ldg_nc_u16(vw + (t + 1) * p.win_ts + ch);
                return __byte_perm(lo, hi, 0x5410);
            };
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c0 = hf * 64 + 8 * tb + j, c1 = c0 + 4;
                    mma16816(dv[hf][j], pair(tA, c0), pair(tA, c1), pair(tA + 8, c0), pair(tA + 8, c1), pb0, pb1);
                }
        }
    }

    if (timed_out && tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_TIMEOUT);

    // ---- epilogue: sum the four warps' partial outputs and write the record (an empty one after a timeout, so
    // that the merge below still sees every record arrive)
    __syncthreads();
#pragma unroll
    for (int hf = 0; hf < 2; ++hf)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c0 = hf * 64 + 8 * tb + j, c1 = c0 + 4;
            if (2 * cp < G) {
                red[(static_cast<size_t>(warp) * G + 2 * cp) * kD + c0] = dv[hf][j][0];
                red[(static_cast<size_t>(warp) * G + 2 * cp) * kD + c1] = dv[hf][j][2];
            }
            if (2 * cp + 1 < G) {
                red[(static_cast<size_t>(warp) * G + 2 * cp + 1) * kD + c0] = dv[hf][j][1];
                red[(static_cast<size_t>(warp) * G + 2 * cp + 1) * kD + c1] = dv[hf][j][3];
            }
        }
    __syncthreads();
    for (int idx = tid; idx < G * kD; idx += kAThreads) {
        const int g = idx / kD, c = idx % kD;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kAWarps; ++w) s += red[(static_cast<size_t>(w) * G + g) * kD + c];
        record_ptr(p, G, h, split, g)[c] = timed_out ? 0.f : s;
    }
#pragma unroll
    for (int j = 0; j < kHeadsPerWarp; ++j) {
        const int g = warp + j * kAWarps;
        if (g < G) {
            const float l = warp_sum_f32(l_run[j]);
            if (lane == 0) {
                float* rec = record_ptr(p, G, h, split, g);
                rec[kPartM] = timed_out ? -INFINITY : m_run[j];
                rec[kPartL] = timed_out ? 0.f : l;
            }
        }
    }

    // ---- merge: the CTA that arrives last at this kv head's counter combines all records
    //      out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
    if (p.counters == nullptr) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned arrived = atomicAdd(p.counters + h, 1u) + 1u;
        s_last = arrived == gridDim.x;
        if (s_last) p.counters[h] = 0u;   // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // warp w merges heads w, w + 4: its lanes fetch the records' (m, l) in parallel, the weights go through shared
    // memory (the reduction buffer is free again), then every lane sums four channels over the records
    const int nrec = p.nrec;
    float* wgt = red;   // [G][nrec], nrec <= 129
    for (int g = warp; g < G; g += kAWarps) {
        const float* base = record_ptr(p, G, h, 0, g);
        const int64_t step = static_cast<int64_t>(p.rec_group) * kPartialStride;
        float M = -INFINITY;
        for (int s = lane; s < nrec; s += 32) M = fmaxf(M, ldcg_f32(base + s * step + kPartM));
        M = warp_max_f32(M);
        float l = 0.f;
        for (int s = lane; s < nrec; s += 32) {
            const float ms = ldcg_f32(base + s * step + kPartM);
            const float w = (ms == -INFINITY) ? 0.f : fast_exp2(ms - M);
            l += w * ldcg_f32(base + s * step + kPartL);
            wgt[g * nrec + s] = w;
        }
        l = warp_sum_f32(l);
        __syncwarp();
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* col = base + 4 * lane;
        int s = 0;
        for (; s + 4 <= nrec; s += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = ldcg_f32x4(col + (s + u) * step);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float w = wgt[g * nrec + s + u];
                o.x += w * v[u].x; o.y += w * v[u].y; o.z += w * v[u].z; o.w += w * v[u].w;
            }
        }
        for (; s < nrec; ++s) {
            const float4 v = ldcg_f32x4(col + s * step);
            const float w = wgt[g * nrec + s];
            o.x += w * v.x; o.y += w * v.y; o.z += w * v.z; o.w += w * v.w;
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __half* dst = p.out + (static_cast<int64_t>(h) * G + g) * p.out_stride + 4 * lane;
        dst[0] = __float2half_rn(o.x * inv);
        dst[1] = __float2half_rn(o.y * inv);
        dst[2] = __float2half_rn(o.z * inv);
        dst[3] = __float2half_rn(o.w * inv);
    }
}

template <int G, int QBITS, bool GROUP32>
static int launch_attn(const DecodeParams& p, int n_kv_heads, int grid_x, cudaStream_t s) {
    const AttnLayout lay(p.cap, G, QBITS ? sizeof(QBuf<QBITS ? QBITS : 2>) : 0);
    static size_t configured[64] = {0};   // largest dynamic shared memory size opted into so far, per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MFAR_ERR_LAUNCH;
    if (lay.total > configured[dev]) {
        if (cudaFuncSetAttribute(decode_attn_kernel<G, QBITS, GROUP32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(lay.total)) != cudaSuccess)
            return MFAR_ERR_LAUNCH;
        configured[dev] = lay.total;
    }
    decode_attn_kernel<G, QBITS, GROUP32><<<dim3(grid_x, n_kv_heads), kAThreads, lay.total, s>>>(p);
    return launch_status();
}

template <int QBITS, bool GROUP32>
static int dispatch_attn(const DecodeParams& p, int G, int n_kv_heads, int grid_x, cudaStream_t s) {
    switch (G) {
        case 1: return launch_attn<1, QBITS, GROUP32>(p, n_kv_heads, grid_x, s);
        case 2: return launch_attn<2, QBITS, GROUP32>(p, n_kv_heads, grid_x, s);
        case 4: return launch_attn<4, QBITS, GROUP32>(p, n_kv_heads, grid_x, s);
        case 8: return launch_attn<8, QBITS, GROUP32>(p, n_kv_heads, grid_x, s);
        default: return MFAR_ERR_ARG;
    }
}

int launch_decode_attn(const DecodeParams& p, int G, int n_kv_heads, int grid_x, cudaStream_t s) {
    return dispatch_attn<0, false>(p, G, n_kv_heads, grid_x, s);
}

int launch_decode_attn_quant(const DecodeParams& p, int G, int bits, bool group32, int n_kv_heads, int grid_x,
                             cudaStream_t s) {
    if (bits == 2) return group32 ? dispatch_attn<2, true>(p, G, n_kv_heads, grid_x, s) : dispatch_attn<2, false>(p, G, n_kv_heads, grid_x, s);
    if (bits == 4) return group32 ? dispatch_attn<4, true>(p, G, n_kv_heads, grid_x, s) : dispatch_attn<4, false>(p, G, n_kv_heads, grid_x, s);
    return MFAR_ERR_ARG;
}

}  // namespace mfar
