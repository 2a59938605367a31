// One-shot all-reduce fused with the residual add and the RMSNorm that follow it in a tensor-parallel decode step:
//     x[row] += sum over ranks of partial_r[row];   out[row] = fp16(x * rsqrt(mean(x^2) + eps)) * weight
// The reference has no distributed code; this replaces the NCCL all-reduce + mfar_add_rmsnorm_f16 pair of the
// tensor-parallel end-to-end model (one [batch, hidden] fp16 partial per rank, 256 KiB at batch 32: latency bound).
//
// Every rank launches the same kernel on its own GPU.  Each rank's partial lives in a buffer that the other ranks
// have mapped (CUDA IPC); the kernel
//   1. announces "my partial of call `epoch` is complete" by storing the epoch into slot [rank] of every peer's flag
//      array (plain system-scope stores over NVLink; the partial was written by the previous kernel on this stream);
//   2. waits until its own flag array shows the epoch for every peer.  The wait is bounded by `wait_ns`: when it runs
//      out the CTA records MFAR_DEV_TIMEOUT and leaves without touching x or out (no trap, the context stays usable).
//      The bit is sticky: launches that find it set still announce, but do not wait again, so a step of 64 reductions
//      replayed from a CUDA graph costs one bound, not 64, before the host sees the error;
//   3. reads the peers' rows with plain L1-bypassing loads through the peer pointers (no TMA, no multicast of any
//      kind), sums them in rank order in fp32 - the same order on every rank, so all ranks get identical bits -
//      adds the residual and normalises.
// Epochs grow monotonically (the caller passes step * calls_per_step + call index, the step read from device memory so
// that a captured launch can be replayed), so flags never need clearing.  Two partial buffers alternate: a rank can
// only finish call k + 1 after every peer has started it, i.e. after every peer has finished reading call k's buffer.
#include "common.cuh"
#include <cstring>

namespace mfar {

constexpr int kMaxPeers = 8;

struct PeerReduceParams {
    const __half* partial[kMaxPeers];   // this call's partial of every rank (peer pointers; [rank] is local)
    unsigned* flags[kMaxPeers];         // flag array (kMaxPeers words) of every rank; [rank] is local
    int world, rank;
    const int* step_dev;                // optional: step counter in device memory
    int step, calls_per_step, call;
    __half* x;
    const __half* w;
    __half* out;
    int hidden;
    float eps;
    unsigned long long wait_ns;
    unsigned* dev_status;
};

__device__ __forceinline__ uint4 ld_peer_u4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys_u32(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_sys_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One CTA per row; hidden / 8 threads (up to 1024), so that with hidden <= 8192 every thread has a single 16-byte piece
// per rank and all its peer loads are in flight together: one NVLink round trip, not one per piece.
__global__ void __launch_bounds__(1024) peer_reduce_rmsnorm_kernel(PeerReduceParams p) {
    __shared__ float red[32];
    __shared__ int s_ok;
    const int tid = threadIdx.x;
    const int step = p.step_dev ? *p.step_dev : p.step;
    const unsigned epoch = static_cast<unsigned>(step) * static_cast<unsigned>(p.calls_per_step) + static_cast<unsigned>(p.call) + 1u;

    // 1. announce (first CTA only; the partial is complete: it was written by an earlier kernel of this stream)
    if (blockIdx.x == 0 && tid < p.world) {
        __threadfence_system();
        st_sys_u32(p.flags[tid] + p.rank, epoch);
    }
    // 2. wait for every peer's announcement of this epoch (or a later one), bounded
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < p.world) {
        const unsigned* f = p.flags[p.rank] + tid;
        const unsigned long long t0 = global_timer_ns();
        // an earlier reduction already gave up: the group is broken, look once and do not wait
        const bool broken = p.dev_status && (ld_volatile_u32(p.dev_status) & MFAR_DEV_TIMEOUT);
        bool ok = !(broken && static_cast<int>(ld_sys_u32(f) - epoch) < 0);
        unsigned spins = 0;
        while (ok && static_cast<int>(ld_sys_u32(f) - epoch) < 0) {
            if ((++spins & 63u) == 0 && global_timer_ns() - t0 > p.wait_ns) ok = false;
        }
        if (!ok) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_TIMEOUT);
        return;
    }

    // 3. sum the partials in rank order, add the residual, normalise
    const int64_t row = blockIdx.x;
    __half* xr = p.x + row * p.hidden;
    float ss = 0.f;
    const int nthr = blockDim.x;
    for (int i = tid * 8; i < p.hidden; i += nthr * 8) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        uint4 v[kMaxPeers];
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r < p.world) v[r] = ld_peer_u4(p.partial[r] + row * p.hidden + i);
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (r < p.world) {
                const __half2* h2 = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = __half22float2(h2[k]);
                    acc[2 * k] += f.x;
                    acc[2 * k + 1] += f.y;
                }
            }
        uint4 a = *reinterpret_cast<const uint4*>(xr + i);
        __half2* ah = reinterpret_cast<__half2*>(&a);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(ah[k]);
            ah[k] = __floats2half2_rn(f.x + acc[2 * k], f.y + acc[2 * k + 1]);
            const float2 g = __half22float2(ah[k]);
            ss += g.x * g.x + g.y * g.y;
        }
        *reinterpret_cast<uint4*>(xr + i) = a;
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) ss += __shfl_xor_sync(kFull, ss, d);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (nthr >> 5); ++i) tot += red[i];
    const float scale = rsqrtf(tot / static_cast<float>(p.hidden) + p.eps);
    __half* orow = p.out + row * p.hidden;
    for (int i = tid * 8; i < p.hidden; i += nthr * 8) {
        const uint4 a = *reinterpret_cast<const uint4*>(xr + i);   // own writes: same thread, same addresses
        const uint4 g = *reinterpret_cast<const uint4*>(p.w + i);
        const __half2* ah = reinterpret_cast<const __half2*>(&a);
        const __half2* gh = reinterpret_cast<const __half2*>(&g);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(ah[k]);
            oh[k] = __hmul2(__floats2half2_rn(f.x * scale, f.y * scale), gh[k]);
        }
        *reinterpret_cast<uint4*>(orow + i) = o;
    }
}

// ---- arg-max over a vocabulary that is split across the ranks (each rank holds the logits of its slice).
// Two launches: row_argmax_kernel leaves (value, global index) of every row's best local logit in this rank's
// peer-visible pair buffer; peer_argmax_exchange_kernel then announces, waits (bounded, like the reduction above),
// reads every rank's pairs through the peer pointers and keeps the best: the largest value, the smallest index among
// equals, so every rank ends up with the same token.
struct ArgPair { float v; int idx; };

__global__ void __launch_bounds__(256) row_argmax_kernel(const __half* logits, int64_t stride, int n, int vocab_offset,
                                                         ArgPair* pairs) {
    __shared__ float s_v[8];
    __shared__ int s_i[8];
    const int tid = threadIdx.x;
    const __half* row = logits + static_cast<int64_t>(blockIdx.x) * stride;
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = tid * 8; i < n; i += 256 * 8) {           // n is a multiple of 8, rows are 16-byte aligned
        const uint4 q = *reinterpret_cast<const uint4*>(row + i);
        const __half2* h2 = reinterpret_cast<const __half2*>(&q);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(h2[k]);
            if (f.x > best) { best = f.x; at = i + 2 * k; }        // ascending indices: the first of equals stays
            if (f.y > best) { best = f.y; at = i + 2 * k + 1; }
        }
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        const float ov = __shfl_xor_sync(kFull, best, d);
        const int oi = __shfl_xor_sync(kFull, at, d);
        if (ov > best || (ov == best && oi < at)) { best = ov; at = oi; }
    }
    if ((tid & 31) == 0) { s_v[tid >> 5] = best; s_i[tid >> 5] = at; }
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int w = 1; w < 8; ++w)
            if (s_v[w] > best || (s_v[w] == best && s_i[w] < at)) { best = s_v[w]; at = s_i[w]; }
        ArgPair r;
        r.v = best;
        r.idx = at == 0x7fffffff ? vocab_offset : vocab_offset + at;
        pairs[blockIdx.x] = r;
    }
}

struct ArgExchangeParams {
    const ArgPair* pairs[kMaxPeers];
    unsigned* flags[kMaxPeers];
    int world, rank;
    const int* step_dev;
    int step, calls_per_step, call, rows;
    long long* tokens;
    unsigned long long wait_ns;
    unsigned* dev_status;
};

__global__ void __launch_bounds__(256) peer_argmax_exchange_kernel(ArgExchangeParams p) {
    __shared__ int s_ok;
    const int tid = threadIdx.x;
    const int step = p.step_dev ? *p.step_dev : p.step;
    const unsigned epoch = static_cast<unsigned>(step) * static_cast<unsigned>(p.calls_per_step) + static_cast<unsigned>(p.call) + 1u;
    if (tid < p.world) {          // this rank's pairs were written by the launch before this one
        __threadfence_system();
        st_sys_u32(p.flags[tid] + p.rank, epoch);
    }
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < p.world) {
        const unsigned* f = p.flags[p.rank] + tid;
        const unsigned long long t0 = global_timer_ns();
        const bool broken = p.dev_status && (ld_volatile_u32(p.dev_status) & MFAR_DEV_TIMEOUT);
        bool ok = !(broken && static_cast<int>(ld_sys_u32(f) - epoch) < 0);
        unsigned spins = 0;
        while (ok && static_cast<int>(ld_sys_u32(f) - epoch) < 0) {
            if ((++spins & 63u) == 0 && global_timer_ns() - t0 > p.wait_ns) ok = false;
        }
        if (!ok) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) {
        if (tid == 0 && p.dev_status) atomicOr(p.dev_status, MFAR_DEV_TIMEOUT);
        return;
    }
    for (int row = tid; row < p.rows; row += 256) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int r = 0; r < p.world; ++r) {
            unsigned long long raw;
            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(raw) : "l"(p.pairs[r] + row) : "memory");
            const float v = __uint_as_float(static_cast<unsigned>(raw));
            const int idx = static_cast<int>(raw >> 32);
            if (v > best || (v == best && idx < at) || at == 0x7fffffff) { best = v; at = idx; }
        }
        p.tokens[row] = at;
    }
}

}  // namespace mfar

using namespace mfar;

// Buffers that peers map.  The mapping has to be opened with the READING GPU current (cudaIpcOpenMemHandle maps into
// the current context and sets up the peer path lazily): a mapping opened in the owner's context of the importing
// process - which is what torch's tensor sharing does - is not reachable from kernels of another GPU.
extern "C" int mfar_peer_alloc(int64_t bytes, void** ptr, void* handle64) {
    if (bytes <= 0 || !ptr || !handle64) return MFAR_ERR_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    void* d = nullptr;
    if (cudaMalloc(&d, static_cast<size_t>(bytes)) != cudaSuccess) { cudaGetLastError(); return MFAR_ERR_WORKSPACE; }
    cudaIpcMemHandle_t h;
    if (cudaMemset(d, 0, static_cast<size_t>(bytes)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&h, d) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(d);
        return MFAR_ERR_LAUNCH;
    }
    memcpy(handle64, &h, sizeof(h));
    *ptr = d;
    return MFAR_OK;
}

extern "C" int mfar_peer_open(const void* handle64, void** ptr) {
    if (!handle64 || !ptr) return MFAR_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* d = nullptr;
    if (cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return MFAR_ERR_LAUNCH; }
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, d) != cudaSuccess || at.type != cudaMemoryTypeDevice) {
        cudaGetLastError();
        cudaIpcCloseMemHandle(d);
        return MFAR_ERR_ARG;
    }
    *ptr = d;
    return MFAR_OK;
}

extern "C" int mfar_peer_close(void* ptr) {
    if (!ptr) return MFAR_OK;
    if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) { cudaGetLastError(); return MFAR_ERR_LAUNCH; }
    return MFAR_OK;
}

extern "C" int mfar_peer_free(void* ptr) {
    if (!ptr) return MFAR_OK;
    if (cudaFree(ptr) != cudaSuccess) { cudaGetLastError(); return MFAR_ERR_LAUNCH; }
    return MFAR_OK;
}

extern "C" int mfar_peer_reduce_add_rmsnorm_f16(void* x, const void* const* partials, void* const* flags, int world,
                                                int rank, const int32_t* step_dev, int step, int calls_per_step,
                                                int call, const void* weight, void* out, int64_t rows, int hidden,
                                                float eps, int64_t wait_ns, uint32_t* dev_status, void* stream) {
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || rows < 0 || hidden <= 0 || (hidden % 8) ||
        calls_per_step <= 0 || call < 0 || call >= calls_per_step || step < 0 || wait_ns <= 0)
        return MFAR_ERR_ARG;
    if (rows == 0) return MFAR_OK;
    if (!x || !partials || !flags || !weight || !out) return MFAR_ERR_ARG;
    if (rows > 0x7fffffffll) return MFAR_ERR_LIMIT;
    PeerReduceParams p{};
    for (int r = 0; r < world; ++r) {
        if (!partials[r] || !flags[r]) return MFAR_ERR_ARG;
        if ((reinterpret_cast<uintptr_t>(partials[r]) & 15) || (reinterpret_cast<uintptr_t>(flags[r]) & 3)) return MFAR_ERR_ALIGN;
        p.partial[r] = static_cast<const __half*>(partials[r]);
        p.flags[r] = static_cast<unsigned*>(flags[r]);
    }
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return MFAR_ERR_ALIGN;
    p.world = world;
    p.rank = rank;
    p.step_dev = step_dev;
    p.step = step;
    p.calls_per_step = calls_per_step;
    p.call = call;
    p.x = static_cast<__half*>(x);
    p.w = static_cast<const __half*>(weight);
    p.out = static_cast<__half*>(out);
    p.hidden = hidden;
    p.eps = eps;
    p.wait_ns = static_cast<unsigned long long>(wait_ns);
    p.dev_status = dev_status;
    const int pieces = hidden / 8;
    const int threads = pieces >= 1024 ? 1024 : ((pieces + 31) / 32) * 32;
    peer_reduce_rmsnorm_kernel<<<static_cast<unsigned>(rows), threads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return launch_status();
}

extern "C" int mfar_peer_argmax_f16(const void* logits, int64_t row_stride, int64_t rows, int n_local, int vocab_offset,
                                    void* const* pairs, void* const* flags, int world, int rank,
                                    const int32_t* step_dev, int step, int calls_per_step, int call, int64_t* tokens,
                                    int64_t wait_ns, uint32_t* dev_status, void* stream) {
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || rows < 0 || n_local <= 0 || (n_local % 8) ||
        vocab_offset < 0 || calls_per_step <= 0 || call < 0 || call >= calls_per_step || step < 0 || wait_ns <= 0)
        return MFAR_ERR_ARG;
    if (rows == 0) return MFAR_OK;
    if (!logits || !pairs || !flags || !tokens) return MFAR_ERR_ARG;
    if (rows > 65535) return MFAR_ERR_LIMIT;
    if ((reinterpret_cast<uintptr_t>(logits) & 15) || (row_stride & 7)) return MFAR_ERR_ALIGN;
    ArgExchangeParams p{};
    for (int r = 0; r < world; ++r) {
        if (!pairs[r] || !flags[r]) return MFAR_ERR_ARG;
        if ((reinterpret_cast<uintptr_t>(pairs[r]) & 7) || (reinterpret_cast<uintptr_t>(flags[r]) & 3)) return MFAR_ERR_ALIGN;
        p.pairs[r] = static_cast<const ArgPair*>(pairs[r]);
        p.flags[r] = static_cast<unsigned*>(flags[r]);
    }
    p.world = world;
    p.rank = rank;
    p.step_dev = step_dev;
    p.step = step;
    p.calls_per_step = calls_per_step;
    p.call = call;
    p.rows = static_cast<int>(rows);
    p.tokens = reinterpret_cast<long long*>(tokens);
    p.wait_ns = static_cast<unsigned long long>(wait_ns);
    p.dev_status = dev_status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    row_argmax_kernel<<<static_cast<unsigned>(rows), 256, 0, s>>>(static_cast<const __half*>(logits), row_stride, n_local,
                                                                 vocab_offset,
                                                                 const_cast<ArgPair*>(p.pairs[rank]));
    const int st = launch_status();
    if (st != MFAR_OK) return st;
    peer_argmax_exchange_kernel<<<1, 256, 0, s>>>(p);
    return launch_status();
}
