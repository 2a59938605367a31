// Pieces shared by the fp16 and the quantised compression kernels: the per-row
// magnitude selector and the decoupled look-back that orders blocks inside a chain.
#pragma once

#include "common.cuh"

namespace mfar {

constexpr int kXsStride = 144;  // halves per shared-memory row: 288 B keeps 16-B chunks conflict free
constexpr unsigned long long kFlagAggregate = 1ull << 62;
constexpr unsigned long long kFlagPrefix = 2ull << 62;
constexpr unsigned long long kValueMask = (1ull << 62) - 1;

// rank-th smallest magnitude among the 128 values held by a thread pair
// (m[] = |x| as packed half2, 32 per thread).  Returns the fp16 bit pattern.
__device__ __forceinline__ unsigned select_threshold(const __half2 (&m)[32], int rank) {
    unsigned T = 0;
#pragma unroll 1
    for (int bit = 14; bit >= 0; --bit) {
        const unsigned short tr = static_cast<unsigned short>(T | ((1u << bit) - 1u));
        const __half2 t2 = __half2half2(__ushort_as_half(tr));
        __half2 c0 = __float2half2_rn(0.f), c1 = c0, c2 = c0, c3 = c0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            c0 = __hadd2(c0, __hle2(m[j + 0], t2));
            c1 = __hadd2(c1, __hle2(m[j + 1], t2));
            c2 = __hadd2(c2, __hle2(m[j + 2], t2));
            c3 = __hadd2(c3, __hle2(m[j + 3], t2));
        }
        c0 = __hadd2(__hadd2(c0, c1), __hadd2(c2, c3));
        int cnt = static_cast<int>(__low2float(c0) + __high2float(c0));
        cnt += __shfl_xor_sync(kFull, cnt, 1);
        if (cnt < rank) T |= (1u << bit);
    }
    return T;
}

// Loads the pair's half of a row (chunks 2j+hh of 8 halves) and prunes it in registers.
// keep_sign: leave the sign bit of pruned elements (what x * 0 gives) instead of +0.
__device__ __forceinline__ void load_prune_row(const __half* row, int hh, int rank, bool keep_sign, uint4 (&v)[8]) {
    const uint4* src = reinterpret_cast<const uint4*>(row);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = ldg_nc_u4(src + 2 * j + hh);
    if (rank <= 0) return;
    __half2 m[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const unsigned w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const unsigned a = w[e] & 0x7fff7fffu;
            m[4 * j + e] = *reinterpret_cast<const __half2*>(&a);
        }
    }
    const unsigned T = select_threshold(m, rank);
    const __half2 t2 = __half2half2(__ushort_as_half(static_cast<unsigned short>(T)));
    const unsigned sign = keep_sign ? 0x80008000u : 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        unsigned* w = reinterpret_cast<unsigned*>(&v[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) w[e] &= (__hge2_mask(m[4 * j + e], t2) | sign);
    }
}

// Exclusive prefix of `total` over the chain of blocks [first, b) whose status words live in
// `st` (indexed by chain position).  Called by one whole warp; every lane returns the same
// value, or -1 after a bounded wait gave up (the error words are set).  The block's own
// inclusive prefix is published in any case so that successors never wait for it.
__device__ __forceinline__ long long lookback_exclusive(unsigned long long* st, int b, int first, unsigned total,
                                                        unsigned* err, unsigned* dev_status) {
    const int lane = threadIdx.x & 31;
    long long excl = 0;
    bool failed = false;
    if (b > first) {
        if (lane == 0) st_volatile_u64(st + b, kFlagAggregate | total);
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
