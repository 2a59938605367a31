// Fused per-token magnitude prune + bitmap + asymmetric low-bit quantised compression.
//
// Same skeleton as compress.cu (one CTA of 128 threads per 64-token block of one head, rows
// pruned in registers by thread pairs, one thread per tile afterwards, decoupled look-back for
// the block's position in the packed stream).  Per tile the thread makes two passes over its
// 64 values in shared memory:
//   pass 1  bitmap, raw count, min / max of the nonzeros of every group
//           -> scale = (max - min) / (2^bits - 1) (1 if that is 0), zero = floor(-min / scale + 0.5),
//              both computed in fp32 and stored fp16;
//   pass 2  codes clamp(floor(v / scale_fp16 + 0.5) + zero_fp16, 0, 2^bits - 1), IEEE division,
//           packed 32/bits per uint32, least significant first.
// bits = 2, group = 64 reproduces kernel_quant/compression_quant.py bit for bit; bits = 4 and
// group = 32 (a fresh scale / zero every 32 nonzeros of a tile) extend it.
#include "compress_common.cuh"

namespace mfar {

struct QuantParams {
    const __half* x;
    int64_t xhs, xts;
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
    __shared__ __align__(16) unsigned short xs[64 * kXsStride];
    __shared__ unsigned ps[128 * 8];
    __shared__ unsigned s_warp[4];
    __shared__ unsigned s_ticket;
    __shared__ long long s_excl;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_ticket = atomicAdd(p.ticket, 1u);
    __syncthreads();
    const int h = static_cast<int>(s_ticket) / p.nblk;
    const int b = static_cast<int>(s_ticket) % p.nblk;
    if (h >= p.n_heads) return;

    {
        const int r = tid >> 1, hh = tid & 1;
        uint4 v[8];
        load_prune_row(p.x + h * p.xhs + (static_cast<int64_t>(b) * 64 + r) * p.xts, hh, p.rank, false, v);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(&xs[r * kXsStride + 8 * (2 * j + hh)]) = v[j];
    }
    __syncthreads();

    // element e of this thread's tile
    const int base = (KIND == MFAR_KIND_KEY) ? tid : ((tid & 63) * kXsStride + (tid >> 6) * 64);
    const int step = (KIND == MFAR_KIND_KEY) ? kXsStride : 1;
    const int maxq = (1 << p.bits) - 1;
    const int cap = 32 / p.bits;
    const int ngrp = 64 / p.group;

    // ---- pass 1
    unsigned hi = 0, lo = 0;
    int cnt = 0;
    float mn[2] = {INFINITY, INFINITY}, mx[2] = {-INFINITY, -INFINITY};
#pragma unroll 8
    for (int e = 0; e < 64; ++e) {
        const unsigned short u = xs[base + e * step];
        const bool nz = (u & 0x7fffu) != 0;
        if (e < 32) hi = (hi << 1) | nz; else lo = (lo << 1) | nz;
        if (nz) {
            const float f = __half2float(__ushort_as_half(u));
            const int g = (ngrp == 2 && cnt >= 32) ? 1 : 0;
            mn[g] = fminf(mn[g], f);
            mx[g] = fmaxf(mx[g], f);
            ++cnt;
        }
    }
    const int64_t tile = p.tile_start + static_cast<int64_t>(b) * kTilesPerBlock + tid;
    const int64_t mi = h * p.meta_hs + tile;
    GroupQ gq[2];
    for (int g = 0; g < ngrp; ++g)
        gq[g] = make_group(mn[g], mx[g], cnt > 32 * g, maxq, &p.scales[mi * ngrp + g], &p.zeros[mi * ngrp + g]);
    const unsigned units = (cnt + cap - 1) / cap;

    // ---- scan of the units, position of the block in the packed stream
    unsigned incl = units;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned n = __shfl_up_sync(kFull, incl, d);
        if (lane >= d) incl += n;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    unsigned wbase = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const unsigned t = s_warp[w];
        if (w < warp) wbase += t;
        total += t;
    }
    incl += wbase;
    const unsigned excl_tile = incl - units;

    // chain: all blocks of all heads when the packed stream is compact, one chain per head otherwise.
    // The block's total is announced now; the look-back itself waits until the codes are packed, by
    // which time the predecessors have announced theirs.
    const bool compact = p.packed_hs == 0;
    const int pos = h * p.nblk + b;
    const int chain_first = compact ? 0 : h * p.nblk;
    if (tid == 0) lookback_announce(p.state, pos, chain_first, total);
    p.bmp[h * p.bmp_hs + tile] = (static_cast<unsigned long long>(hi) << 32) | lo;
    if (p.counts) p.counts[mi] = cnt;
    if (p.units) p.units[mi] = static_cast<int>(units);

    // ---- pass 2: codes, packed in shared memory in final order
    {
        unsigned word = 0, o = excl_tile;
        int k = 0;
#pragma unroll 8
        for (int e = 0; e < 64; ++e) {
            const unsigned short u = xs[base + e * step];
            if ((u & 0x7fffu) != 0) {
                const GroupQ& g = gq[(ngrp == 2 && k >= 32) ? 1 : 0];
                const float f = __half2float(__ushort_as_half(u));
                float q = __fadd_rn(floorf(__fadd_rn(__fdiv_rn(f, g.scale), 0.5f)), g.zero);
                q = fminf(fmaxf(q, 0.f), static_cast<float>(maxq));
                word |= static_cast<unsigned>(q) << ((k % cap) * p.bits);
                ++k;
                if (k % cap == 0) { ps[o++] = word; word = 0; }
            }
        }
        if (k % cap) ps[o++] = word;
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
    p.tile_off[mi] = static_cast<int>(blk_start + excl_tile);
    if (blk_start + total > limit) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_CAPACITY);
        return;
    }
    for (unsigned i = tid; i < total; i += 128) p.packed[blk_start + i] = ps[i];
}

// arena mode: head_tail[h] += words appended (separate tiny launch so that no block reads a moved tail)
__global__ void quant_bump_tails(const unsigned long long* state, int nblk, int n_heads, int* head_tail) {
    const int h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h < n_heads) head_tail[h] += static_cast<int>(state[static_cast<int64_t>(h) * nblk + nblk - 1] & kValueMask);
}

}  // namespace mfar

using namespace mfar;

extern "C" int mfar_compress_quant(const void* x, int64_t x_head_stride, int64_t x_token_stride, int n_heads,
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
