// Shared device helpers for the sm_100a sparse KV-cache kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mustafar_b200.h"

namespace mfar {

constexpr int kD = MFAR_HEAD_DIM;            // channels per head
constexpr int kBlockTokens = MFAR_BLOCK_TOKENS;
constexpr int kTilesPerBlock = MFAR_TILES_PER_BLOCK;
constexpr unsigned kFull = 0xffffffffu;

// Every wait on a flag or an mbarrier is bounded by wall time: after this many
// nanoseconds the kernel records MFAR_DEV_TIMEOUT and leaves.
constexpr unsigned long long kWaitLimitNs = 500ull * 1000ull * 1000ull;

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned lane_id() { return threadIdx.x & 31u; }

__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint4 ldg_nc_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ unsigned warp_sum_u32(unsigned v) { return __reduce_add_sync(kFull, v); }

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

// multiprocessors of the current device (queried once per device; api_misc.cu)
int device_sm_count();

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? MFAR_OK : MFAR_ERR_LAUNCH; }

}  // namespace mfar
