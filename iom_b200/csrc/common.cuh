// Shared device/host helpers of the iom_b200 kernels (sm_100a only).
//
// Layout facts used throughout (reference: src/tensor.cpp:136-164): the last
// two dimensions are stored as 16x16 tiles, tile-row major inside a plane, and
// a tile is 256 consecutive slots (row in tile, then column in tile). A tile is
// therefore 512 bytes for 16-bit leaves and 1024 bytes for 32-bit leaves, one
// in-tile row is 32 / 64 contiguous bytes, and a 16-row band of a plane is one
// contiguous run of tile_columns tiles.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/iom_b200.h"

namespace iomb {

constexpr uint32_t kTile = 16;
constexpr uint32_t kTileSlots = 256;
constexpr uint32_t kMaxLead = IOMB_MAX_LEADING;

// Thread-local error text behind iomb_last_error().
void set_error(const char* text);
int fail(int status, const char* text);
int check_launch(const char* what);
// Names the kernel instance a dispatcher chose, behind iomb_last_launch().
void note_launch(const char* text);

// Number of SMs of the current device (cached per device ordinal).
int sm_count();

// One operand as the kernels see it: plane mapping aligned to the (collapsed)
// leading axes of the operation, zero stride on broadcast axes.
struct Operand {
    unsigned char* base;
    uint64_t plane0;
    uint64_t stride[kMaxLead];
    uint32_t tile_rows;   // tile rows of this operand's own matrix
    uint32_t tile_cols;   // tile columns of this operand's own matrix
    uint32_t bc_rows;     // operand has one row, the result has more
    uint32_t bc_cols;     // operand has one column, the result has more
};

// Collapsed leading iteration space shared by all operands of one launch.
struct Leading {
    uint32_t count;
    uint32_t contiguous;  // every operand advances by exactly one plane per index
    uint64_t dims[kMaxLead];
    uint64_t planes;      // product of dims
};

// Owner plane of logical plane `index` for one operand.
__device__ __forceinline__ uint64_t operand_plane(
        const Operand& operand, const Leading& leading, uint64_t index) {
    uint64_t plane = operand.plane0;
    if (leading.count == 1) {
        return plane + index * operand.stride[0];
    }
    for (int axis = static_cast<int>(leading.count) - 1; axis >= 0; --axis) {
        const uint64_t extent = leading.dims[axis];
        const uint64_t coordinate = index % extent;
        index /= extent;
        plane += coordinate * operand.stride[axis];
    }
    return plane;
}

// ---- numeric helpers ------------------------------------------------------

// BF16 pair packed in one 32-bit word -> two binary32 values (exact widening).
__device__ __forceinline__ float bf16_lo(uint32_t word) {
    return __uint_as_float(word << 16);
}
__device__ __forceinline__ float bf16_hi(uint32_t word) {
    return __uint_as_float(word & 0xFFFF0000u);
}

// Every NaN half of a packed BF16 pair becomes the positive quiet NaN 0x7FC0 (the
// reference's canonical encoding, src/shared/scalar_binary_codec.hpp:79-85); other halves
// pass. One packed unordered compare gives an all-ones mask per NaN half, one logic
// operation selects: no branch.
__device__ __forceinline__ uint32_t canonical_bf16x2(uint32_t word) {
    uint32_t nan_halves;
    asm("set.nan.u32.bf16x2 %0, %1, %1;" : "=r"(nan_halves) : "r"(word));
    return (word & ~nan_halves) | (nan_halves & 0x7FC07FC0u);
}

// Two binary32 values -> packed BF16 pair, round-to-nearest-even, overflow to
// infinity, gradual underflow; every NaN becomes 0x7FC0.
__device__ __forceinline__ uint32_t pack_bf16x2_canonical(float lo, float hi) {
    const __nv_bfloat162 packed = __floats2bfloat162_rn(lo, hi);
    return canonical_bf16x2(*reinterpret_cast<const uint32_t*>(&packed));
}

// Packed BF16 arithmetic: the sm_100a packed instructions (add/sub/mul.rn.bf16x2: the
// exact result rounded once to BF16, subnormals kept). Building with
// -DIOMB_PACKED_BF16=0 gives each half one binary32 operation and one RNE narrowing
// instead. Both are the reference codec's result: the binary32 detour is a double
// rounding that cannot change a BF16 result (24 >= 2*8 + 2); the tests run every pair of
// BF16 codes through the kernels against the codec.
#ifndef IOMB_PACKED_BF16
#define IOMB_PACKED_BF16 1
#endif
__device__ __forceinline__ uint32_t add_bf16x2_canonical(uint32_t a, uint32_t b) {
#if IOMB_PACKED_BF16
    uint32_t r;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return canonical_bf16x2(r);
#else
    return pack_bf16x2_canonical(__fadd_rn(bf16_lo(a), bf16_lo(b)),
                                 __fadd_rn(bf16_hi(a), bf16_hi(b)));
#endif
}
__device__ __forceinline__ uint32_t sub_bf16x2_canonical(uint32_t a, uint32_t b) {
#if IOMB_PACKED_BF16
    uint32_t r;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return canonical_bf16x2(r);
#else
    return pack_bf16x2_canonical(__fsub_rn(bf16_lo(a), bf16_lo(b)),
                                 __fsub_rn(bf16_hi(a), bf16_hi(b)));
#endif
}
__device__ __forceinline__ uint32_t mul_bf16x2_canonical(uint32_t a, uint32_t b) {
#if IOMB_PACKED_BF16
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return canonical_bf16x2(r);
#else
    return pack_bf16x2_canonical(__fmul_rn(bf16_lo(a), bf16_lo(b)),
                                 __fmul_rn(bf16_hi(a), bf16_hi(b)));
#endif
}

// Plain RNE pack for values known not to be NaN.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 packed = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&packed);
}

__device__ __forceinline__ uint32_t f32_canonical_bits(float value) {
    return value != value ? 0x7FC00000u : __float_as_uint(value);
}

__device__ __forceinline__ uint4 load_u4(const void* address) {
    return *reinterpret_cast<const uint4*>(address);
}
__device__ __forceinline__ uint4 load_u4_stream(const void* address) {
    return __ldcs(reinterpret_cast<const uint4*>(address));
}
__device__ __forceinline__ void store_u4(void* address, uint4 value) {
    *reinterpret_cast<uint4*>(address) = value;
}
__device__ __forceinline__ void store_u4_stream(void* address, uint4 value) {
    __stcs(reinterpret_cast<uint4*>(address), value);
}
// A load that asks L2 to keep the line (for data read again and again, such as an embedding
// table, beside a stream that would otherwise push it out).
__device__ __forceinline__ uint64_t l2_keep_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ uint4 load_u4_keep(const void* address, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(address), "l"(policy));
    return v;
}
// 256-bit streaming accesses (sm_100): 32-byte-aligned address, one instruction
// for two neighbouring 16-byte vectors.
__device__ __forceinline__ void load_u8_stream(const void* address, uint4* lo, uint4* hi) {
    asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(lo->x), "=r"(lo->y), "=r"(lo->z), "=r"(lo->w), "=r"(hi->x), "=r"(hi->y),
                   "=r"(hi->z), "=r"(hi->w)
                 : "l"(address));
}
__device__ __forceinline__ void store_u8_stream(void* address, uint4 lo, uint4 hi) {
    asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(address), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y),
                    "r"(hi.z), "r"(hi.w)
                 : "memory");
}

}  // namespace iomb
