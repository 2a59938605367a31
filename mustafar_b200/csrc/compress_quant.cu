// Fused per-token magnitude prune + bitmap + asymmetric low-bit quantised compression.
//
// Same skeleton as compress.cu (one CTA of 128 threads per 64-token block of one head, the row
// selection leaves one "kept and nonzero" flag per element, the flags become the bitmaps, decoupled
// look-back for the block's position in the packed stream).  Then:
//   1. the kept values go to shared memory in tile order, unpadded;
//   2. one thread per tile takes min / max of every group of its values
//      -> scale = (max - min) / (2^bits - 1) (1 if that is 0), zero = floor(-min / scale + 0.5),
//         both computed in fp32 and stored fp16;
//   3. the block's values are dealt out evenly over the threads (tiles differ wildly in size: a K
//      outlier channel keeps all 64 tokens, most keep ~20), each computes
//      clamp(floor(v / scale_fp16 + 0.5) + zero_fp16, 0, 2^bits - 1), IEEE division, and ors its
//      code into the tile's word: 32/bits codes per uint32, least significant first.
// bits = 2, group = 64 reproduces kernel_quant/compression_quant.py bit for bit; bits = 4 and
// group = 32 (a fresh scale / zero every 32 nonzeros of a tile) extend it.
#include "compress_common.cuh"

namespace mfar {

struct QuantParams {
    const __half* x;
    int64_t xhs, xts;
    int hpg;                       // heads per group (0: one stride for all heads)
    int64_t xgs;                   // stride between groups of heads
    int n_heads, nblk, rank, bits, group;
    unsigned long long* bmp;
    int* tile_off;
    int* counts;
    int* units;
    __half* scales;
    __half* zeros;
    int64_t bmp_hs, meta_hs, tile_start;
    unsigned* packed;
    int64_t packed_hs, packed_cap;
    int* head_tail;
    unsigned* ticket;
    unsigned* err;
    unsigned long long* state;
    unsigned* dev_status;
};

struct GroupQ {
    float scale, zero;   // the fp16-rounded parameters, widened again
};

__device__ __forceinline__ GroupQ make_group(float xmin, float xmax, bool has, int maxq, __half* s_out, __half* z_out) {
    float scale = 1.f, zero = 0.f;
    if (has) {
        scale = __fdiv_rn(__fsub_rn(xmax, xmin), static_cast<float>(maxq));
        if (scale == 0.f) scale = 1.f;
        zero = floorf(__fadd_rn(__fdiv_rn(-xmin, scale), 0.5f));
    }
    const __half sh = __float2half_rn(scale), zh = __float2half_rn(zero);
    *s_out = sh;
    *z_out = zh;
    GroupQ g;
    g.scale = __half2float(sh);
    if (g.scale == 0.f) g.scale = 1.f;
    g.zero = __half2float(zh);
    return g;
}

template <int KIND>
__global__ void __launch_bounds__(128) compress_quant_kernel(QuantParams p) {
    __shared__ __align__(16) unsigned short vals[64 * 128];                                     // kept values, tile order, no padding
    __shared__ __align__(16) unsigned short xs[KIND == MFAR_KIND_KEY ? 64 * kXsStride : 8];     // K: the raw block
    __shared__ unsigned s_mask[4][64];       // K: keep flags [32-channel word][row], first channel in the top bit
    __shared__ unsigned s_voff[129];         // first value of every tile in vals (and the total)
    __shared__ unsigned s_woff[129];         // first code word of every tile in words (and the total)
    __shared__ float4 s_par[128];            // per tile: scale, zero of group 0, scale, zero of group 1 (fp16 values, widened)
    __shared__ unsigned words[128 * 8];      // code words of the block, final order
    __shared__ unsigned s_warp[4][2];
    __shared__ unsigned s_ticket;
    __shared__ long long s_excl;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int r = tid >> 1, hh = tid & 1;    // row of the block and member of the pair that owns it
    if (tid == 0) s_ticket = atomicAdd(p.ticket, 1u);
    __syncthreads();
    const int h = static_cast<int>(s_ticket) / p.nblk;
    const int b = static_cast<int>(s_ticket) % p.nblk;
    if (h >= p.n_heads) return;
    const int maxq = (1 << p.bits) - 1;
    const int cap = 32 / p.bits;
    const int ngrp = 64 / p.group;

    // ---- the pair loads one row, selects the threshold, ends up with one "kept and nonzero" flag per element
    uint4 v[8];
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.x + (p.hpg > 0 ? (h / p.hpg) * p.xgs + (h % p.hpg) * p.xhs : h * p.xhs) + (static_cast<int64_t>(b) * 64 + r) * p.xts);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = ldg_nc_u4(src + 2 * j + hh);
    }
    const unsigned (&w)[32] = reinterpret_cast<const unsigned (&)[32]>(v);
    if (KIND == MFAR_KIND_KEY) {
#pragma unroll
        for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(&xs[r * kXsStride + 8 * (2 * j + hh)]) = v[j];
    }
    const RowSelect sel = select_row(w, p.rank);
    const unsigned y0 = plane_to_bitmap_order(sel.keep0), y1 = plane_to_bitmap_order(sel.keep1);
    const unsigned q0 = __shfl_xor_sync(kFull, y0, 1), q1 = __shfl_xor_sync(kFull, y1, 1);
    unsigned hi0, lo0, hi1, lo1;
    interleave_chunk_bytes(hh ? q0 : y0, hh ? y0 : q0, hi0, lo0);   // channels 0..63
    interleave_chunk_bytes(hh ? q1 : y1, hh ? y1 : q1, hi1, lo1);   // channels 64..127
#pragma unroll
    for (int j = 0; j < 8; ++j) words[tid + 128 * j] = 0;

    // ---- bitmap, count and code words of the tile this thread answers for; both running sums in one scan
    // (values in the low half, words in the high half: at most 8192 and 1024 per block)
    unsigned hi, lo;
    int tile;
    if (KIND == MFAR_KIND_KEY) {
        if (hh == 0) {
            s_mask[0][r] = hi0;
            s_mask[1][r] = lo0;
        } else {
            s_mask[2][r] = hi1;
            s_mask[3][r] = lo1;
        }
        __syncthreads();
        hi = __brev(warp_transpose32(__brev(s_mask[warp][lane])));
        lo = __brev(warp_transpose32(__brev(s_mask[warp][32 + lane])));
        tile = tid;
    } else {
        hi = hh ? hi1 : hi0;
        lo = hh ? lo1 : lo0;
        tile = hh * 64 + r;
    }
    const int cnt = __popc(hi) + __popc(lo);
    const unsigned units = (cnt + cap - 1) / cap;
    const unsigned both = static_cast<unsigned>(cnt) | (units << 16);
    unsigned incl = both;
#pragma unroll
    for (int d = (KIND == MFAR_KIND_KEY ? 1 : 2); d < 32; d <<= 1) {
        const unsigned n = __shfl_up_sync(kFull, incl, d);
        if (lane >= d) incl += n;
    }
    if (KIND == MFAR_KIND_KEY) {
        if (lane == 31) s_warp[warp][0] = incl;
    } else if (lane >= 30) {
        s_warp[warp][hh] = incl;
    }
    __syncthreads();
    unsigned all = 0;
    {
        unsigned half0 = 0;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            const unsigned t0 = s_warp[wi][0], t1 = (KIND == MFAR_KIND_KEY) ? 0u : s_warp[wi][1];
            if (wi < warp) incl += (KIND == MFAR_KIND_VALUE && hh) ? t1 : t0;
            half0 += t0;
            all += t0 + t1;
        }
        if (KIND == MFAR_KIND_VALUE && hh) incl += half0;   // all of channel half 0 comes before half 1
    }
    const unsigned excl = incl - both;
    const unsigned voff = excl & 0xffffu, woff = excl >> 16;
    const unsigned total_vals = all & 0xffffu, total = all >> 16;
    s_voff[tile] = voff;
    s_woff[tile] = woff;
    if (tid == 0) {
        s_voff[128] = total_vals;
        s_woff[128] = total;
    }

    // chain: all blocks of all heads when the packed stream is compact, one chain per head otherwise.
    // The block's total is announced now; the look-back itself waits until the codes are packed, by
    // which time the predecessors have announced theirs.
    const bool compact = p.packed_hs == 0;
    const int pos = h * p.nblk + b;
    const int chain_first = compact ? 0 : h * p.nblk;
    if (tid == 0) lookback_announce(p.state, pos, chain_first, total);

    // ---- kept values into vals, tile order (K: down the columns of the raw block; V: from the registers)
    if (KIND == MFAR_KIND_KEY) {
        unsigned o = voff;
        const int c = tid;
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if ((hi >> (31 - i)) & 1u) vals[o++] = xs[i * kXsStride + c];
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if ((lo >> (31 - i)) & 1u) vals[o++] = xs[(32 + i) * kXsStride + c];
    } else {
        const unsigned voff_other = __shfl_xor_sync(kFull, voff, 1);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const unsigned thi = t ? hi1 : hi0, tlo = t ? lo1 : lo0, y = t ? y1 : y0;
            const unsigned long long bm = (static_cast<unsigned long long>(thi) << 32) | tlo;
            const unsigned off = (hh == t) ? voff : voff_other;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int cidx = 2 * k + hh;                        // chunk inside the tile
                unsigned o = off + (cidx ? __popcll(bm >> (64 - 8 * cidx)) : 0);
                const unsigned flags = y >> (24 - 8 * k);           // bit 7 = first element of the chunk
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const unsigned word = w[16 * t + 4 * k + (e >> 1)];
                    if ((flags >> (7 - e)) & 1u) vals[o++] = static_cast<unsigned short>((e & 1) ? (word >> 16) : word);
                }
            }
        }
    }
    __syncthreads();

    // ---- per tile: min / max of every group -> scale, zero (fp32 arithmetic, stored fp16).  One thread per
    // tile; dealing the values out evenly with shared-memory min / max on ordered keys measured slower.
    const int64_t gtile = p.tile_start + static_cast<int64_t>(b) * kTilesPerBlock + tile;
    const int64_t mi = h * p.meta_hs + gtile;
    {
        float mn0 = INFINITY, mx0 = -INFINITY, mn1 = INFINITY, mx1 = -INFINITY;
        const int n0 = (ngrp == 2 && cnt > 32) ? 32 : cnt;
        for (int k = 0; k < n0; ++k) {
            const float f = __half2float(__ushort_as_half(vals[voff + k]));
            mn0 = fminf(mn0, f);
            mx0 = fmaxf(mx0, f);
        }
        for (int k = n0; k < cnt; ++k) {
            const float f = __half2float(__ushort_as_half(vals[voff + k]));
            mn1 = fminf(mn1, f);
            mx1 = fmaxf(mx1, f);
        }
        const GroupQ g0 = make_group(mn0, mx0, cnt > 0, maxq, &p.scales[mi * ngrp], &p.zeros[mi * ngrp]);
        GroupQ g1;
        g1.scale = 1.f;
        g1.zero = 0.f;
        if (ngrp == 2) g1 = make_group(mn1, mx1, cnt > 32, maxq, &p.scales[mi * 2 + 1], &p.zeros[mi * 2 + 1]);
        s_par[tile] = make_float4(g0.scale, g0.zero, g1.scale, g1.zero);
    }
    __syncthreads();

    // ---- codes: the block's values are dealt out evenly, a contiguous run per thread (tiles differ wildly in
    // size: a K outlier channel keeps all 64 tokens, most keep ~20); each code is or-ed into its tile's word
    {
        const unsigned per = (total_vals + 127u) >> 7;
        const unsigned run0 = tid * per, run1 = min(run0 + per, total_vals);
        if (run0 < run1) {
            int t = 0;   // tile of the first value: largest t with s_voff[t] <= run0
#pragma unroll
            for (int step = 64; step; step >>= 1)
                if (t + step < 128 && s_voff[t + step] <= run0) t += step;
            unsigned base_t = s_voff[t], next = s_voff[t + 1];
            for (unsigned i = run0; i < run1; ++i) {
                while (i >= next) {   // also skips empty tiles
                    ++t;
                    base_t = next;
                    next = s_voff[t + 1];
                }
                const unsigned k = i - base_t;
                const float4 par = s_par[t];
                const bool g1 = (ngrp == 2 && k >= 32u);
                const float scale = g1 ? par.z : par.x, zero = g1 ? par.w : par.y;
                const float f = __half2float(__ushort_as_half(vals[i]));
                float q = __fadd_rn(floorf(__fadd_rn(__fdiv_rn(f, scale), 0.5f)), zero);
                q = fminf(fmaxf(q, 0.f), static_cast<float>(maxq));
                atomicOr(&words[s_woff[t] + k / cap], static_cast<unsigned>(q) << ((k % cap) * p.bits));
            }
        }
    }

    if (warp == 0) {
        const long long e = lookback_exclusive(p.state, pos, chain_first, total, p.err, p.dev_status, false);
        if (lane == 0) s_excl = e;
    }
    __syncthreads();
    if (s_excl < 0) return;

    long long blk_start;   // uint32 offset in the flat packed buffer
    long long limit;
    if (compact) {
        blk_start = s_excl;
        limit = p.packed_cap;
        if (p.head_tail && b == p.nblk - 1 && tid == 0) p.head_tail[h] = static_cast<int>(blk_start + total);
    } else {
        // (in arena mode head_tail[h] is bumped by quant_bump_tails after this kernel, so every
        // block of the head reads the same, old, tail)
        const long long tail = p.head_tail ? p.head_tail[h] : 0;
        blk_start = h * p.packed_hs + tail + s_excl;
        limit = h * p.packed_hs + p.packed_cap;
    }
    p.bmp[h * p.bmp_hs + gtile] = (static_cast<unsigned long long>(hi) << 32) | lo;
    p.tile_off[mi] = static_cast<int>(blk_start + woff);
    if (p.counts) p.counts[mi] = cnt;
    if (p.units) p.units[mi] = static_cast<int>(units);
    if (blk_start + total > limit) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_CAPACITY);
        return;
    }
    for (unsigned i = tid; i < total; i += 128) p.packed[blk_start + i] = words[i];
}

// arena mode: head_tail[h] += words appended (separate tiny launch so that no block reads a moved tail)
__global__ void quant_bump_tails(const unsigned long long* state, int nblk, int n_heads, int* head_tail) {
    const int h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h < n_heads) head_tail[h] += static_cast<int>(state[static_cast<int64_t>(h) * nblk + nblk - 1] & kValueMask);
}

}  // namespace mfar

using namespace mfar;

extern "C" int mfar_compress_quant(const void* x, int64_t x_head_stride, int64_t x_token_stride,
                                   int heads_per_group, int64_t x_group_stride, int n_heads,
                                   int n_tokens, int kind, int prune_rank, int bits, int group,
                                   int64_t* bitmaps, int64_t bmp_head_stride, int32_t* tile_offsets,
                                   int32_t* counts, int32_t* units, void* scales, void* zeros,
                                   int64_t meta_head_stride, int64_t tile_start, int32_t* packed,
                                   int64_t packed_head_stride, int64_t packed_capacity, int32_t* head_tail,
                                   void* scratch, size_t scratch_bytes, uint32_t* dev_status, void* stream) {
    if (n_heads < 0 || n_tokens < 0 || (n_tokens % 64) != 0) return MFAR_ERR_ARG;
    if (kind != MFAR_KIND_KEY && kind != MFAR_KIND_VALUE) return MFAR_ERR_ARG;
    if ((bits != 2 && bits != 4) || (group != 32 && group != 64)) return MFAR_ERR_ARG;
    if (prune_rank < 0 || prune_rank > kD || tile_start < 0 || (tile_start % kTilesPerBlock) != 0) return MFAR_ERR_ARG;
    if (packed_head_stride < 0 || (packed_head_stride > 0 && !head_tail)) return MFAR_ERR_ARG;
    if (n_heads == 0 || n_tokens == 0) return MFAR_OK;
    if (!x || !bitmaps || !tile_offsets || !scales || !zeros || !packed || !scratch) return MFAR_ERR_ARG;
    if (heads_per_group > 0 && (x_group_stride & 7)) return MFAR_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (x_head_stride & 7) || (x_token_stride & 7) ||
        (reinterpret_cast<uintptr_t>(scratch) & 15) || (reinterpret_cast<uintptr_t>(packed) & 3))
        return MFAR_ERR_ALIGN;
    const size_t need = mfar_compress_scratch_bytes(n_heads, n_tokens);
    if (scratch_bytes < need) return MFAR_ERR_WORKSPACE;
    const int nblk = n_tokens / 64;
    if (static_cast<int64_t>(n_heads) * nblk > 0x7fffffffll) return MFAR_ERR_LIMIT;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(scratch, 0, need, s) != cudaSuccess) return MFAR_ERR_LAUNCH;

    QuantParams p;
    p.x = static_cast<const __half*>(x);
    p.xhs = x_head_stride;
    p.xts = x_token_stride;
    p.hpg = heads_per_group > 0 ? heads_per_group : 0;
    p.xgs = x_group_stride;
    p.n_heads = n_heads;
    p.nblk = nblk;
    p.rank = prune_rank;
    p.bits = bits;
    p.group = group;
    p.bmp = reinterpret_cast<unsigned long long*>(bitmaps);
    p.tile_off = tile_offsets;
    p.counts = counts;
    p.units = units;
    p.scales = static_cast<__half*>(scales);
    p.zeros = static_cast<__half*>(zeros);
    p.bmp_hs = bmp_head_stride;
    p.meta_hs = meta_head_stride;
    p.tile_start = tile_start;
    p.packed = reinterpret_cast<unsigned*>(packed);
    p.packed_hs = packed_head_stride;
    p.packed_cap = packed_capacity;
    p.head_tail = head_tail;
    p.ticket = static_cast<unsigned*>(scratch);
    p.err = p.ticket + 1;
    p.state = reinterpret_cast<unsigned long long*>(static_cast<char*>(scratch) + 16);
    p.dev_status = dev_status;

    const unsigned grid = static_cast<unsigned>(n_heads) * static_cast<unsigned>(nblk);
    if (kind == MFAR_KIND_KEY)
        compress_quant_kernel<MFAR_KIND_KEY><<<grid, 128, 0, s>>>(p);
    else
        compress_quant_kernel<MFAR_KIND_VALUE><<<grid, 128, 0, s>>>(p);
    int r = launch_status();
    if (r) return r;
    if (packed_head_stride > 0) {
        quant_bump_tails<<<(n_heads + 127) / 128, 128, 0, s>>>(p.state, nblk, n_heads, head_tail);
        r = launch_status();
    }
    return r;
}
