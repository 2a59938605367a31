// Pure bit manipulation used by the compression kernels (no memory, no warp communication), kept
// apart so that a host build can check it: define MFAR_BITS_FN and the three intrinsics it uses
// (__byte_perm, __brev, __popc) before including this file outside nvcc.
#pragma once

#ifndef MFAR_BITS_FN
#define MFAR_BITS_FN __device__ __forceinline__
#endif

namespace mfar {

// Transposes, in place, the two 16x16 bit matrices that the low and the high halves of a[0..15] form:
// afterwards bit j (bit 16+j) of a[b] is bit b of the low (high) half of the old a[j].  Recursive block
// swap: bytes by prmt, then nibbles, bit pairs and bits by shift + bit-select (112 instructions).
MFAR_BITS_FN void transpose16x16x2(unsigned (&a)[16]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const unsigned x = a[i], y = a[i + 8];
        a[i] = __byte_perm(x, y, 0x6240);
        a[i + 8] = __byte_perm(x, y, 0x7351);
    }
#pragma unroll
    for (int s = 4; s >= 1; s >>= 1) {
        const unsigned M = s == 4 ? 0x0f0f0f0fu : (s == 2 ? 0x33333333u : 0x55555555u);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (i & s) continue;
            const unsigned x = a[i], y = a[i + s];
            a[i] = (x & M) | ((y << s) & ~M);
            a[i + s] = ((x >> s) & M) | (y & ~M);
        }
    }
}

// A plane word of transpose16x16x2 holds one flag per element of 16 registers: bit j for the low half
// of register j, bit 16+j for its high half.  Sixteen registers are four 16-byte chunks of a row, so
// element e = 0..31 of those chunks (memory order) sits at bit (e >> 1) + 16 * (e & 1).  This returns
// the same flags in bitmap order: element e at bit 31 - e (first element in the top bit), i.e. one
// byte per chunk, first chunk in the top byte.  Perfect shuffle of the two halves, then bit reversal.
MFAR_BITS_FN unsigned plane_to_bitmap_order(unsigned x) {
    x = __byte_perm(x, 0u, 0x3120);
    x = (x & 0xf00ff00fu) | ((x & 0x0f000f00u) >> 4) | ((x & 0x00f000f0u) << 4);
    x = (x & 0xc3c3c3c3u) | ((x & 0x30303030u) >> 2) | ((x & 0x0c0c0c0cu) << 2);
    x = (x & 0x99999999u) | ((x & 0x44444444u) >> 1) | ((x & 0x22222222u) << 1);
    return __brev(x);
}

// A thread pair splits a row's sixteen chunks alternately (member hh owns chunks hh, 2+hh, ...).
// even / odd: bitmap-order words of the even and the odd member for the same eight chunks (one byte
// per chunk, first chunk on top).  Returns the 64-bit bitmap of those eight chunks in memory order.
MFAR_BITS_FN void interleave_chunk_bytes(unsigned even, unsigned odd, unsigned& hi, unsigned& lo) {
    hi = __byte_perm(even, odd, 0x3726);   // [e3 o3 e2 o2]
    lo = __byte_perm(even, odd, 0x1504);   // [e1 o1 e0 o0]
}

}  // namespace mfar
