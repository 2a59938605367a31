// Pieces shared by the fp16 and the quantised compression kernels: the per-row
// magnitude selector and the decoupled look-back that orders blocks inside a chain.
#pragma once

#include "common.cuh"
#include "compress_bits.cuh"

namespace mfar {

constexpr int kXsStride = 144;  // halves per shared-memory row: 288 B keeps 16-B chunks conflict free
constexpr unsigned long long kFlagAggregate = 1ull << 62;
constexpr unsigned long long kFlagPrefix = 2ull << 62;
constexpr unsigned long long kValueMask = (1ull << 62) - 1;

// Result of the per-row selection for one member of the thread pair that owns the row.
struct RowSelect {
    unsigned T;             // fp16 bit pattern of the rank-th smallest magnitude (same in both members)
    unsigned keep0, keep1;  // plane-layout flags (see plane_to_bitmap_order) of the member's chunks 0..3 and
                            // 4..7: the element survives pruning AND is not zero
};

// rank-th smallest magnitude (1-based) among the 128 values held by a thread pair; w[] = the pair
// member's 64 halves (sign bits ignored).  rank <= 0: no pruning (T = 0, every nonzero kept).
//
// Bit-sliced radix select: the 64 magnitudes are transposed into 15 bit planes of 2 x 32 elements
// (element order inside a plane does not matter for counting), then the threshold is built from
// the top bit down: `cand` marks the elements whose higher bits equal the threshold so far; if at
// least `rank` of them have a 0 in this bit the threshold has a 0 there too and the ones are known
// to be greater, else the zeros are smaller than the answer and leave, taking their count off the
// rank.  Per step: 2 and-not, 2 popc and one shuffle to join the pair, instead of 64 compare/add
// on packed halves.  What is greater than or still equal to the threshold at the end is kept.
__device__ __forceinline__ RowSelect select_row(const unsigned (&w)[32], int rank) {
    unsigned p0[16], p1[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        p0[j] = w[j] & 0x7fff7fffu;
        p1[j] = w[16 + j] & 0x7fff7fffu;
    }
    transpose16x16x2(p0);
    transpose16x16x2(p1);
    unsigned c0 = kFull, c1 = kFull, g0 = 0, g1 = 0, T = 0;
    if (rank > 0) {
        int r = rank;
#pragma unroll
        for (int b = 14; b >= 0; --b) {
            const unsigned z0 = c0 & ~p0[b], z1 = c1 & ~p1[b];
            int cnt = __popc(z0) + __popc(z1);
            cnt += __shfl_xor_sync(kFull, cnt, 1);
            const bool zero_side = r <= cnt;
            const unsigned o0 = c0 ^ z0, o1 = c1 ^ z1;   // candidates with a 1 in this bit
            g0 |= zero_side ? o0 : 0u;
            g1 |= zero_side ? o1 : 0u;
            c0 = zero_side ? z0 : o0;
            c1 = zero_side ? z1 : o1;
            if (!zero_side) {
                r -= cnt;
                T |= 1u << b;
            }
        }
    }
    RowSelect res;
    res.T = T;
    res.keep0 = g0 | c0;
    res.keep1 = g1 | c1;
    if (T == 0) {   // zeros pass a zero threshold but never enter a bitmap
        unsigned n0 = 0, n1 = 0;
#pragma unroll
        for (int b = 0; b < 15; ++b) {
            n0 |= p0[b];
            n1 |= p1[b];
        }
        res.keep0 &= n0;
        res.keep1 &= n1;
    }
    return res;
}

__device__ __forceinline__ unsigned select_threshold(const unsigned (&w)[32], int rank) { return select_row(w, rank).T; }

// 32 x 32 bit transpose across a warp: lane i passes row i, lane j returns column j (bit i = bit j of lane i's x).
__device__ __forceinline__ unsigned warp_transpose32(unsigned x) {
    const unsigned lane = lane_id();
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        const unsigned m = s == 16 ? 0x0000ffffu : s == 8 ? 0x00ff00ffu : s == 4 ? 0x0f0f0f0fu : s == 2 ? 0x33333333u : 0x55555555u;
        const unsigned y = __shfl_xor_sync(kFull, x, s);
        x = (lane & s) ? (((y >> s) & m) | (x & ~m)) : ((x & m) | ((y << s) & ~m));
    }
    return x;
}

// Loads the pair's half of a row (chunks 2j+hh of 8 halves) and prunes it in registers.
// keep_sign: leave the sign bit of pruned elements (what x * 0 gives) instead of +0.
__device__ __forceinline__ void load_prune_row(const __half* row, int hh, int rank, bool keep_sign, uint4 (&v)[8]) {
    const uint4* src = reinterpret_cast<const uint4*>(row);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = ldg_nc_u4(src + 2 * j + hh);
    if (rank <= 0) return;
    unsigned (&w)[32] = reinterpret_cast<unsigned (&)[32]>(v);
    const unsigned T = select_threshold(w, rank);
    const __half2 t2 = __half2half2(__ushort_as_half(static_cast<unsigned short>(T)));
    const unsigned sign = keep_sign ? 0x80008000u : 0u;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const unsigned a = w[j] & 0x7fff7fffu;
        w[j] &= (__hge2_mask(*reinterpret_cast<const __half2*>(&a), t2) | sign);
    }
}

// Early half of the look-back, for kernels that have other work to do before they need their prefix:
// one thread announces the block's total as soon as it is known (the chain's first block can publish
// its inclusive prefix right away); lookback_exclusive(..., publish_aggregate = false) follows later.
__device__ __forceinline__ void lookback_announce(unsigned long long* st, int b, int first, unsigned total) {
    // max, not store: a warp of the same CTA may already have published the inclusive prefix, which ranks higher
    atomicMax(st + b, (b > first ? kFlagAggregate : kFlagPrefix) | total);
}

// Waits until the shared-memory counter `c` (bumped by other warps of the same CTA) reaches `target`.
// Called by a whole warp: lane 0 polls, everybody gets the verdict.  False after the wall-time limit.
__device__ __forceinline__ bool wait_shared_counter(const unsigned* c, unsigned target) {
    bool ok = true;
    if (lane_id() == 0) {
        const volatile unsigned* vc = c;
        unsigned spins = 0;
        unsigned long long t0 = 0;
        while (static_cast<int>(*vc - target) < 0) {
            if ((++spins & 255u) == 0) {
                const unsigned long long now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > kWaitLimitNs) {
                    ok = false;
                    break;
                }
            }
            __nanosleep(20);
        }
        __threadfence_block();
    }
    return __shfl_sync(kFull, ok ? 1 : 0, 0) != 0;
}

// Exclusive prefix of `total` over the chain of blocks [first, b) whose status words live in
// `st` (indexed by chain position).  Called by one whole warp; every lane returns the same
// value, or -1 after a bounded wait gave up (the error words are set).  The block's own
// inclusive prefix is published in any case so that successors never wait for it.
__device__ __forceinline__ long long lookback_exclusive(unsigned long long* st, int b, int first, unsigned total,
                                                        unsigned* err, unsigned* dev_status,
                                                        bool publish_aggregate = true) {
    const int lane = threadIdx.x & 31;
    long long excl = 0;
    bool failed = false;
    if (b > first) {
        if (publish_aggregate && lane == 0) st_volatile_u64(st + b, kFlagAggregate | total);
        int j = b - 1;
        while (true) {
            const int idx = j - lane;
            unsigned long long w = kFlagPrefix;  // virtual predecessor of the chain's first block: prefix 0
            if (idx >= first) {
                unsigned spins = 0;
                unsigned long long t0 = 0;
                while (true) {
                    w = ld_volatile_u64(st + idx);
                    if (w >> 62) break;
                    if ((++spins & 255u) == 0) {
                        const unsigned long long now = global_timer_ns();
                        if (t0 == 0) t0 = now;
                        if (now - t0 > kWaitLimitNs || ld_volatile_u32(err)) {
                            failed = true;
                            break;
                        }
                    }
                    __nanosleep(32);
                }
            }
            if (__any_sync(kFull, failed)) { failed = true; break; }
            const unsigned pm = __ballot_sync(kFull, (w >> 62) == 2ull);
            const int firstp = pm ? (__ffs(pm) - 1) : 32;
            const unsigned val = (lane <= firstp) ? static_cast<unsigned>(w & kValueMask) : 0u;
            excl += warp_sum_u32(val);
            if (pm) break;
            j -= 32;
        }
    }
    if (lane == 0) {
        if (failed) {
            atomicOr(err, MFAR_DEV_TIMEOUT);
            if (dev_status) atomicOr(dev_status, MFAR_DEV_TIMEOUT);
        }
        st_volatile_u64(st + b, kFlagPrefix | static_cast<unsigned long long>(excl + total));
    }
    return failed ? -1ll : excl;
}

}  // namespace mfar
