// Fused per-token magnitude prune + bitmap / packed-value compression (fp16 format).
//
// One CTA (128 threads) owns one 64-token block of one head: 64 rows x 128 channels.
//   1. each thread pair loads one 256-byte row straight into registers,
//   2. finds the rank-th smallest magnitude of the row by a bit-sliced radix select (two
//      16x16 bit transposes per thread, then 15 steps of and-not / popc / one shuffle) and
//      comes out with one "kept and nonzero" flag per element; no pruned copy is made,
//   3. the flags become the bitmaps: a V tile (64 channels of one token) is the pair's own
//      flags, byte-interleaved; a K tile (one channel down 64 tokens) comes from a warp-wide
//      32x32 bit transpose of the block's flag matrix,
//   4. padded counts are scanned inside the CTA; the block's start inside its head comes
//      from a decoupled look-back over the preceding blocks of the same head,
//   5. kept values are packed in shared memory in final order (V: from the registers that
//      loaded them; K: down the columns of the raw block in shared memory) and leave with
//      128-bit coalesced stores.
// CTAs take (head, block) from an atomic ticket, head-major, so every predecessor a
// look-back waits for has already started; the wait is bounded all the same.
#include "compress_common.cuh"

namespace mfar {

// resident CTAs per SM the register allocation aims at.  K tiles: 5 (96 registers; at 6 the bit planes spill and the
// kernel is 20 % slower).  V tiles: 6 (80 registers, 4 bytes of spill, 6 % faster: the V pack works from registers
// and has no column walk that the spill could delay).
constexpr int kCompressMinCtasKey = 5;
constexpr int kCompressMinCtasValue = 6;

struct CompressParams {
    const __half* x;
    int64_t xhs, xts;
    int hpg;                       // heads per group (0: one stride for all heads)
    int64_t xgs;                   // stride between groups of heads
    int n_heads, nblk, rank;
    unsigned long long* bmp;
    int64_t bmp_hs;
    int* acc;
    int64_t acc_hs, tile_start;
    __half* nz;
    const int* nz_off;
    int64_t nz_hs, nz_cap;
    unsigned* ticket;              // scratch[0]
    unsigned* err;                 // scratch[1]
    unsigned long long* state;     // scratch + 16 bytes: one word per (head, block)
    unsigned* dev_status;
    unsigned* max_block;           // optional: running max of packed halves per block
};

template <int KIND>
__global__ void __launch_bounds__(128, KIND == MFAR_KIND_KEY ? kCompressMinCtasKey : kCompressMinCtasValue) compress_kernel(CompressParams p) {
    __shared__ __align__(16) unsigned short ps[64 * 128];                                       // packed values, final order
    __shared__ __align__(16) unsigned short xs[KIND == MFAR_KIND_KEY ? 64 * kXsStride : 8];     // K: the raw block
    __shared__ unsigned s_mask[4][64];         // K: keep flags [32-channel word][row], first channel in the top bit
    __shared__ unsigned s_warp[4][2];
    __shared__ unsigned s_ticket;
    __shared__ long long s_excl;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int r = tid >> 1, hh = tid & 1;      // row of the block and member of the pair that owns it
    const unsigned n_blocks = static_cast<unsigned>(p.n_heads) * static_cast<unsigned>(p.nblk);

    // (head, block) pairs come from an atomic ticket, fetched when the CTA is ready to start on it: blocks
    // then start in ticket order, and a look-back never waits for a predecessor that has not begun.
    {
        if (tid == 0) s_ticket = atomicAdd(p.ticket, 1u);
        __syncthreads();
        const unsigned ticket = s_ticket;
        if (ticket >= n_blocks) return;
        const int h = static_cast<int>(ticket / static_cast<unsigned>(p.nblk));
        const int b = static_cast<int>(ticket % static_cast<unsigned>(p.nblk));

        // ---- 1+2: the pair loads one row (member hh takes chunks hh, 2+hh, ...), selects the
        // threshold and ends up with one flag per element: kept and nonzero
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
        // flags in bitmap order, one byte per chunk; with the partner's they give the row's two 64-bit masks
        const unsigned y0 = plane_to_bitmap_order(sel.keep0), y1 = plane_to_bitmap_order(sel.keep1);
        const unsigned q0 = __shfl_xor_sync(kFull, y0, 1), q1 = __shfl_xor_sync(kFull, y1, 1);
        unsigned hi0, lo0, hi1, lo1;
        interleave_chunk_bytes(hh ? q0 : y0, hh ? y0 : q0, hi0, lo0);   // channels 0..63
        interleave_chunk_bytes(hh ? q1 : y1, hh ? y1 : q1, hi1, lo1);   // channels 64..127

        // ---- 3+4a: bitmap and padded count of the tile this thread answers for, offsets inside the block
        unsigned hi, lo, pad, incl, total;
        int tile;                                  // index of that tile inside the block
        if (KIND == MFAR_KIND_KEY) {
            // tile = channel tid down the 64 rows: transpose the block's flag matrix, 32 x 32 bits per warp step
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
            const unsigned nnz = __popc(hi) + __popc(lo);
            pad = ((nnz + 7u) & ~7u) >> 1;         // uint32 units, reference counts
            incl = pad;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const unsigned n = __shfl_up_sync(kFull, incl, d);
                if (lane >= d) incl += n;
            }
            if (lane == 31) s_warp[warp][0] = incl;
            __syncthreads();
            total = 0;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const unsigned t = s_warp[wi][0];
                if (wi < warp) incl += t;
                total += t;
            }
        } else {
            // tile = (channel half hh, row r), index hh * 64 + r: scan over the rows for each half
            // (lanes two apart), all of half 0 comes before half 1
            hi = hh ? hi1 : hi0;
            lo = hh ? lo1 : lo0;
            tile = hh * 64 + r;
            const unsigned nnz = __popc(hi) + __popc(lo);
            pad = ((nnz + 7u) & ~7u) >> 1;
            incl = pad;
#pragma unroll
            for (int d = 2; d < 32; d <<= 1) {
                const unsigned n = __shfl_up_sync(kFull, incl, d);
                if (lane >= d) incl += n;
            }
            if (lane >= 30) s_warp[warp][hh] = incl;
            __syncthreads();
            unsigned half0 = 0;
            total = 0;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const unsigned t0 = s_warp[wi][0], t1 = s_warp[wi][1];
                if (wi < warp) incl += hh ? t1 : t0;
                half0 += t0;
                total += t0 + t1;
            }
            if (hh) incl += half0;
        }
        const unsigned excl_tile = incl - pad;
        unsigned long long* chain = p.state + static_cast<int64_t>(h) * p.nblk;
        if (tid == 0) lookback_announce(chain, b, 0, total);

        // ---- 5: pack in shared memory in final order (needs no global offset yet)
        if (KIND == MFAR_KIND_KEY) {
            unsigned o = 2 * excl_tile;
            const unsigned end = 2 * incl;
            const int c = tid;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if ((hi >> (31 - i)) & 1u) ps[o++] = xs[i * kXsStride + c];
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if ((lo >> (31 - i)) & 1u) ps[o++] = xs[(32 + i) * kXsStride + c];
            while (o < end) ps[o++] = 0;
        } else {
            // straight from the registers: this member's chunks of both tiles of row r
            const unsigned excl_other = __shfl_xor_sync(kFull, excl_tile, 1);
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const unsigned thi = t ? hi1 : hi0, tlo = t ? lo1 : lo0, y = t ? y1 : y0;
                const unsigned long long bm = (static_cast<unsigned long long>(thi) << 32) | tlo;
                const unsigned off = 2 * (hh == t ? excl_tile : excl_other);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int cidx = 2 * k + hh;                        // chunk inside the tile
                    unsigned o = off + (cidx ? __popcll(bm >> (64 - 8 * cidx)) : 0);
                    const unsigned flags = y >> (24 - 8 * k);           // bit 7 = first element of the chunk
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const unsigned word = w[16 * t + 4 * k + (e >> 1)];
                        if ((flags >> (7 - e)) & 1u) ps[o++] = static_cast<unsigned short>((e & 1) ? (word >> 16) : word);
                    }
                }
                if (hh == t) {   // the tile's owner zero-fills up to the padded length
                    const unsigned n = __popcll(bm);
                    for (unsigned o = off + n; o < off + ((n + 7u) & ~7u); ++o) ps[o] = 0;
                }
            }
        }

        // ---- 4b: start of this block inside its head (decoupled look-back, warp 0; the predecessors
        // announced their totals a pack phase ago)
        if (warp == 0) {
            const long long e = lookback_exclusive(chain, b, 0, total, p.err, p.dev_status, false);
            if (lane == 0) s_excl = e;
        }
        __syncthreads();
        if (s_excl < 0) return;

        const int64_t tile0 = p.tile_start + static_cast<int64_t>(b) * kTilesPerBlock;
        int* acc = p.acc + h * p.acc_hs;
        const long long base = (p.tile_start > 0) ? static_cast<long long>(acc[p.tile_start]) : 0ll;
        const long long blk_start = base + s_excl;  // uint32 units inside the head

        p.bmp[h * p.bmp_hs + tile0 + tile] = (static_cast<unsigned long long>(hi) << 32) | lo;
        acc[tile0 + tile + 1] = static_cast<int>(blk_start + incl);
        if (p.tile_start == 0 && b == 0 && tid == 0) acc[0] = 0;
        if (tid == 0 && p.max_block) atomicMax(p.max_block, 2u * total);

        if (2 * (blk_start + total) > p.nz_cap) {
            // the values of this block are dropped; later blocks still run
            if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_CAPACITY);
        } else {
            __half* head_nz = p.nz + (p.nz_off ? 8ll * p.nz_off[h] : h * p.nz_hs);
            uint4* dst = reinterpret_cast<uint4*>(head_nz + 2 * blk_start);
            const uint4* src = reinterpret_cast<const uint4*>(ps);
            const int n16 = static_cast<int>(total >> 2);
            for (int i = tid; i < n16; i += 128) dst[i] = src[i];
        }
    }
}

__global__ void __launch_bounds__(128) prune_kernel(const __half* x, __half* y, int64_t n_rows,
                                                    int64_t row_stride, int rank) {
    int64_t pair = (static_cast<int64_t>(blockIdx.x) * 128 + threadIdx.x) >> 1;
    const int hh = threadIdx.x & 1;
    // threads past the end redo the last row (no store) so that every warp stays whole for the shuffles
    const bool valid = pair < n_rows;
    if (!valid) pair = n_rows - 1;
    uint4 v[8];
    load_prune_row(x + pair * row_stride, hh, rank, true, v);
    if (!valid) return;
    uint4* dst = reinterpret_cast<uint4*>(y + pair * row_stride);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[2 * j + hh] = v[j];
}

// Packed values of all heads back to back (the reference's torch.cat of per-head buffers): head h, whose values
// lie at nz + h * nz_hs, goes to out + sum of the lengths of the heads before it.  Lengths come from the accum tails
// on the device; grid (chunks, heads), every CTA sums the lengths in front of its head itself.
__global__ void __launch_bounds__(256) compact_heads_kernel(const __half* nz, int64_t nz_hs, const int* acc, int64_t acc_hs,
                                                            int64_t tiles, __half* out, int64_t out_cap) {
    __shared__ long long s_part[8];
    const int h = blockIdx.y;
    long long before = 0;
    for (int j = threadIdx.x; j < h; j += 256) before += 2ll * acc[j * acc_hs + tiles];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) before += __shfl_xor_sync(kFull, before, d);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = before;
    __syncthreads();
    before = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) before += s_part[w];
    const long long len = 2ll * acc[h * acc_hs + tiles];
    if (before + len > out_cap) return;        // never write past the caller's buffer
    const uint4* src = reinterpret_cast<const uint4*>(nz + h * nz_hs);
    uint4* dst = reinterpret_cast<uint4*>(out + before);
    const long long n16 = len >> 3;
    for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < n16; i += static_cast<long long>(gridDim.x) * 256)
        dst[i] = src[i];
}

}  // namespace mfar

using namespace mfar;

extern "C" int mfar_compact_heads_fp16(const void* nz, int64_t nz_head_stride, const int32_t* accum,
                                       int64_t acc_head_stride, int64_t n_tiles, int n_heads, void* out,
                                       int64_t out_capacity, void* stream) {
    if (n_heads < 0 || n_tiles < 0 || out_capacity < 0) return MFAR_ERR_ARG;
    if (n_heads == 0 || out_capacity == 0) return MFAR_OK;
    if (!nz || !accum || !out) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(nz) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) || (nz_head_stride & 7))
        return MFAR_ERR_ALIGN;
    if (n_heads > 65535) return MFAR_ERR_LIMIT;
    int chunks = (device_sm_count() * 8 + n_heads - 1) / n_heads;
    if (chunks < 1) chunks = 1;
    compact_heads_kernel<<<dim3(chunks, n_heads), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(nz), nz_head_stride, accum, acc_head_stride, n_tiles, static_cast<__half*>(out),
        out_capacity);
    return launch_status();
}

extern "C" size_t mfar_compress_scratch_bytes(int n_heads, int n_tokens) {
    if (n_heads <= 0 || n_tokens <= 0) return 16;
    const size_t nblk = (static_cast<size_t>(n_tokens) + 63) / 64;
    return 16 + 8 * static_cast<size_t>(n_heads) * nblk;
}

extern "C" int mfar_compress_fp16(const void* x, int64_t x_head_stride, int64_t x_token_stride,
                                  int heads_per_group, int64_t x_group_stride,
                                  int n_heads, int n_tokens, int kind, int prune_rank,
                                  int64_t* bitmaps, int64_t bmp_head_stride,
                                  int32_t* accum, int64_t acc_head_stride, int64_t tile_start,
                                  void* nz, const int32_t* nz_offset, int64_t nz_head_stride,
                                  int64_t nz_capacity, void* scratch, size_t scratch_bytes,
                                  uint32_t* dev_status, uint32_t* max_block_halves, void* stream) {
    if (n_heads < 0 || n_tokens < 0 || (n_tokens % 64) != 0) return MFAR_ERR_ARG;
    if (kind != MFAR_KIND_KEY && kind != MFAR_KIND_VALUE) return MFAR_ERR_ARG;
    if (prune_rank < 0 || prune_rank > kD || tile_start < 0 || (tile_start % kTilesPerBlock) != 0) return MFAR_ERR_ARG;
    if (n_heads == 0 || n_tokens == 0) return MFAR_OK;
    if (!x || !bitmaps || !accum || !nz || !scratch) return MFAR_ERR_ARG;
    if (heads_per_group > 0 && (x_group_stride & 7)) return MFAR_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (x_head_stride & 7) || (x_token_stride & 7) ||
        (reinterpret_cast<uintptr_t>(nz) & 15) || (nz_head_stride & 7) ||
        (reinterpret_cast<uintptr_t>(scratch) & 15) || (reinterpret_cast<uintptr_t>(bitmaps) & 7) ||
        (reinterpret_cast<uintptr_t>(accum) & 3))
        return MFAR_ERR_ALIGN;
    const size_t need = mfar_compress_scratch_bytes(n_heads, n_tokens);
    if (scratch_bytes < need) return MFAR_ERR_WORKSPACE;
    const int nblk = n_tokens / 64;
    if (static_cast<int64_t>(n_heads) * nblk > 0x7fffffffll) return MFAR_ERR_LIMIT;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(scratch, 0, need, s) != cudaSuccess) return MFAR_ERR_LAUNCH;

    CompressParams p;
    p.x = static_cast<const __half*>(x);
    p.xhs = x_head_stride;
    p.xts = x_token_stride;
    p.hpg = heads_per_group > 0 ? heads_per_group : 0;
    p.xgs = x_group_stride;
    p.n_heads = n_heads;
    p.nblk = nblk;
    p.rank = prune_rank;
    p.bmp = reinterpret_cast<unsigned long long*>(bitmaps);
    p.bmp_hs = bmp_head_stride;
    p.acc = accum;
    p.acc_hs = acc_head_stride;
    p.tile_start = tile_start;
    p.nz = static_cast<__half*>(nz);
    p.nz_off = nz_offset;
    p.nz_hs = nz_head_stride;
    p.nz_cap = nz_capacity;
    p.ticket = static_cast<unsigned*>(scratch);
    p.err = p.ticket + 1;
    p.state = reinterpret_cast<unsigned long long*>(static_cast<char*>(scratch) + 16);
    p.dev_status = dev_status;
    p.max_block = max_block_halves;

    const unsigned n_blocks = static_cast<unsigned>(n_heads) * static_cast<unsigned>(nblk);
    const unsigned grid = n_blocks;
    if (kind == MFAR_KIND_KEY)
        compress_kernel<MFAR_KIND_KEY><<<grid, 128, 0, s>>>(p);
    else
        compress_kernel<MFAR_KIND_VALUE><<<grid, 128, 0, s>>>(p);
    return launch_status();
}

extern "C" int mfar_prune_fp16(const void* x, void* y, int64_t n_rows, int64_t row_stride,
                               int prune_rank, void* stream) {
    if (n_rows < 0 || prune_rank < 0 || prune_rank > kD) return MFAR_ERR_ARG;
    if (n_rows == 0) return MFAR_OK;
    if (!x || !y) return MFAR_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15) || (row_stride & 7))
        return MFAR_ERR_ALIGN;
    const int64_t blocks = (n_rows * 2 + 127) / 128;
    if (blocks > 0x7fffffffll) return MFAR_ERR_LIMIT;
    prune_kernel<<<static_cast<unsigned>(blocks), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<__half*>(y), n_rows, row_stride, prune_rank);
    return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of mfar_compress_fp16.
//
// Some hosts may not call cudaMalloc at all while they run: an inference server whose device
// memory is handed out once at start-up by its own arena, or a plugin that lives inside another
// runtime's memory budget and has nowhere to keep a scratch buffer of its own.  For those callers
// the ticket counter and the per-block status words of the look-back live in a fixed array inside
// this library's device image instead of a caller-provided buffer.
//
// The array costs kStaticScratchBytes of device memory on every GPU that loads the library, for
// as long as the process lives.  It bounds the job size: n_heads * (n_tokens / 64) must not exceed
// MFAR_NOALLOC_MAX_BLOCKS, otherwise MFAR_ERR_LIMIT is returned and nothing is launched.
//
// All calls on one device share the array.  Each call first clears the part it uses (on `stream`),
// so leftovers of an earlier call never matter; two calls that may overlap on the GPU (different
// streams without an ordering between them) would corrupt each other's tickets and must not be issued.
//
// The first call on a device looks the array's device address up (cudaGetSymbolAddress with that
// device current) and remembers it; make that first call outside any stream capture.
constexpr size_t kStaticScratchBytes = 16 + 8 * static_cast<size_t>(MFAR_NOALLOC_MAX_BLOCKS);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static void* g_static_scratch_addr[64] = {nullptr};   // per device; a host-side name is not a device address

extern "C" int mfar_compress_fp16_noalloc(const void* x, int64_t x_head_stride, int64_t x_token_stride,
                                          int n_heads, int n_tokens, int kind, int prune_rank,
                                          int64_t* bitmaps, int64_t bmp_head_stride,
                                          int32_t* accum, int64_t acc_head_stride, int64_t tile_start,
                                          void* nz, const int32_t* nz_offset, int64_t nz_head_stride,
                                          int64_t nz_capacity, uint32_t* dev_status, uint32_t* max_block_halves,
                                          void* stream) {
    if (n_heads < 0 || n_tokens < 0 || (n_tokens % 64) != 0) return MFAR_ERR_ARG;
    if (static_cast<int64_t>(n_heads) * (n_tokens / 64) > MFAR_NOALLOC_MAX_BLOCKS) return MFAR_ERR_LIMIT;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MFAR_ERR_LAUNCH;
    if (g_static_scratch_addr[dev] == nullptr) {
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_static_scratch) != cudaSuccess || addr == nullptr) return MFAR_ERR_LAUNCH;
        g_static_scratch_addr[dev] = addr;
    }
    return mfar_compress_fp16(x, x_head_stride, x_token_stride, 0, 0, n_heads, n_tokens, kind, prune_rank, bitmaps,
                              bmp_head_stride, accum, acc_head_stride, tile_start, nz, nz_offset, nz_head_stride,
                              nz_capacity, g_static_scratch_addr[dev], kStaticScratchBytes, dev_status,
                              max_block_halves, stream);
}
