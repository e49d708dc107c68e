// Pieces shared by the two RMS normalization kernels (rmsnorm.cu: rows of up to
// 2048 values and the sequential order; rmsnorm_long.cu: longer rows).
//
// Arithmetic (src/cpu/queue.cpp:1145-1244): FP32 sum of individually rounded
// squares over the logical features only, mean = sum / F, + eps, true sqrt and
// true division, (x * inv) * w with both products rounded, NaN sign cleared, one
// RNE encode.
#pragma once

#include "host.hpp"

namespace iomb {

struct RmsParams {
    Operand x;
    Operand residual;   // fused only
    Operand sum;        // fused only
    Operand out;
    const unsigned char* scale_row;   // first tile of the [1,F] scale plane
    Leading leading;
    uint32_t rows;
    uint32_t cols;
    uint32_t tile_rows;
    uint32_t tile_cols;
    uint32_t group_rows;        // g
    uint32_t groups_per_band;   // 16 / g
    uint64_t units;             // units of this launch
    uint64_t first_unit;        // first unit of this launch (long rows are launched in parts)
    float eps;
    uint32_t order;
};

__device__ __forceinline__ void cp_async_16(void* shared_dst, const void* global_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(global_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}
// Waits until at most PENDING of this thread's committed groups are in flight.
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(PENDING) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

template <int ELEM>
__device__ __forceinline__ float decode_element(const unsigned char* bytes) {
    if constexpr (ELEM == 2) {
        return __uint_as_float(
                static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(bytes)) << 16);
    } else {
        return *reinterpret_cast<const float*>(bytes);
    }
}

// sum + x*x with both operations rounded (never contracted).
__device__ __forceinline__ float accumulate_square(float sum, float value) {
    return __fadd_rn(sum, __fmul_rn(value, value));
}

// The fixed tree that combines a row's 16 column accumulators
// (src/cpu/avx512_bf16_rmsnorm_reduction.cpp:69-81).
__device__ __forceinline__ float combine_lanes(const float* l) {
    float total[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        total[j] = __fadd_rn(__fadd_rn(__fadd_rn(l[j], l[j + 4]), l[j + 8]), l[j + 12]);
    }
    return __fadd_rn(__fadd_rn(total[0], total[2]), __fadd_rn(total[1], total[3]));
}

// 1 / sqrt(sum / F + eps): true division, true square root, true division.
__device__ __forceinline__ float row_inverse(float sum, uint32_t cols, float eps) {
    const float mean = __fdiv_rn(sum, static_cast<float>(cols));
    const float root = __fsqrt_rn(__fadd_rn(mean, eps));
    return __fdiv_rn(1.0f, root);
}

// With a finite, not vanishing sum every |x * inv| stays near sqrt(F) at most, so
// (x * inv) * w cannot be a NaN for finite w and the canonical-NaN fix-up can be
// skipped for the whole row.
__device__ __forceinline__ bool row_is_clean(float sum, bool scale_finite) {
    return sum >= 5.421010862e-20f && sum <= 3.402823466e+38f && scale_finite;
}

// x + residual for one 16-byte vector, rounded to the leaf, NaNs canonical.
template <int ELEM>
__device__ __forceinline__ uint4 add_vectors(uint4 a, uint4 b) {
    if constexpr (ELEM == 2) {
        return make_uint4(add_bf16x2_canonical(a.x, b.x), add_bf16x2_canonical(a.y, b.y),
                          add_bf16x2_canonical(a.z, b.z), add_bf16x2_canonical(a.w, b.w));
    } else {
        auto word = [](uint32_t p, uint32_t q) {
            return f32_canonical_bits(__fadd_rn(__uint_as_float(p), __uint_as_float(q)));
        };
        return make_uint4(word(a.x, b.x), word(a.y, b.y), word(a.z, b.z), word(a.w, b.w));
    }
}

// One 16-byte vector of raw scale values widened to binary32.
template <int ELEM>
__device__ __forceinline__ void widen_vector(uint4 raw, float* w) {
    if constexpr (ELEM == 2) {
        w[0] = bf16_lo(raw.x); w[1] = bf16_hi(raw.x); w[2] = bf16_lo(raw.y); w[3] = bf16_hi(raw.y);
        w[4] = bf16_lo(raw.z); w[5] = bf16_hi(raw.z); w[6] = bf16_lo(raw.w); w[7] = bf16_hi(raw.w);
    } else {
        w[0] = __uint_as_float(raw.x); w[1] = __uint_as_float(raw.y);
        w[2] = __uint_as_float(raw.z); w[3] = __uint_as_float(raw.w);
    }
}

// (x * inv) * w for one 16-byte vector of x, both products rounded, one RNE encode;
// `fast` skips the canonical-NaN fix-up for rows that cannot produce a NaN.
template <int ELEM>
__device__ __forceinline__ uint4 normalize_vector(uint4 xv, const float* w, float inv, bool fast) {
    if constexpr (ELEM == 2) {
        const float r0 = __fmul_rn(__fmul_rn(bf16_lo(xv.x), inv), w[0]);
        const float r1 = __fmul_rn(__fmul_rn(bf16_hi(xv.x), inv), w[1]);
        const float r2 = __fmul_rn(__fmul_rn(bf16_lo(xv.y), inv), w[2]);
        const float r3 = __fmul_rn(__fmul_rn(bf16_hi(xv.y), inv), w[3]);
        const float r4 = __fmul_rn(__fmul_rn(bf16_lo(xv.z), inv), w[4]);
        const float r5 = __fmul_rn(__fmul_rn(bf16_hi(xv.z), inv), w[5]);
        const float r6 = __fmul_rn(__fmul_rn(bf16_lo(xv.w), inv), w[6]);
        const float r7 = __fmul_rn(__fmul_rn(bf16_hi(xv.w), inv), w[7]);
        if (fast) {
            return make_uint4(pack_bf16x2(r0, r1), pack_bf16x2(r2, r3), pack_bf16x2(r4, r5),
                              pack_bf16x2(r6, r7));
        }
        return make_uint4(pack_bf16x2_canonical(r0, r1), pack_bf16x2_canonical(r2, r3),
                          pack_bf16x2_canonical(r4, r5), pack_bf16x2_canonical(r6, r7));
    } else {
        const float r0 = __fmul_rn(__fmul_rn(__uint_as_float(xv.x), inv), w[0]);
        const float r1 = __fmul_rn(__fmul_rn(__uint_as_float(xv.y), inv), w[1]);
        const float r2 = __fmul_rn(__fmul_rn(__uint_as_float(xv.z), inv), w[2]);
        const float r3 = __fmul_rn(__fmul_rn(__uint_as_float(xv.w), inv), w[3]);
        if (fast) {
            return make_uint4(__float_as_uint(r0), __float_as_uint(r1), __float_as_uint(r2),
                              __float_as_uint(r3));
        }
        return make_uint4(f32_canonical_bits(r0), f32_canonical_bits(r1), f32_canonical_bits(r2),
                          f32_canonical_bits(r3));
    }
}

template <int ELEM>
__device__ __forceinline__ void store_vector_masked(
        unsigned char* address, uint4 value, uint32_t valid) {
    constexpr uint32_t kPerVector = 16 / ELEM;
    if (valid >= kPerVector) {
        store_u4_stream(address, value);
        return;
    }
    const uint32_t words[4] = {value.x, value.y, value.z, value.w};
    for (uint32_t e = 0; e < valid; ++e) {
        if constexpr (ELEM == 4) {
            reinterpret_cast<uint32_t*>(address)[e] = words[e];
        } else {
            reinterpret_cast<uint16_t*>(address)[e] =
                    static_cast<uint16_t>(words[e / 2] >> ((e & 1u) * 16));
        }
    }
}

// Where unit u lives: band (tile row, logical plane) and first in-tile row.
struct RmsUnit {
    uint32_t tr;
    uint32_t row0;
    uint32_t rows_in_band;
    uint64_t index;
    bool valid;
};

// 16 / G groups per band is a power of two; the band arithmetic is 32-bit
// whenever the band count allows (64-bit division costs a hundred instructions
// on every CTA's critical path).
template <int G>
__device__ __forceinline__ RmsUnit rms_locate(const RmsParams& p, uint64_t u) {
    constexpr uint32_t kGroupsPerBand = kTile / G;
    RmsUnit at;
    const uint32_t group = static_cast<uint32_t>(u % kGroupsPerBand);
    const uint64_t band = u / kGroupsPerBand;
    if (band <= 0xFFFFFFFFull) {
        const uint32_t band32 = static_cast<uint32_t>(band);
        at.tr = band32 % p.tile_rows;
        at.index = band32 / p.tile_rows;
    } else {
        at.tr = static_cast<uint32_t>(band % p.tile_rows);
        at.index = band / p.tile_rows;
    }
    at.row0 = group * G;
    at.rows_in_band = min(kTile, p.rows - at.tr * kTile);
    at.valid = at.row0 < at.rows_in_band;     // uniform per CTA
    return at;
}

// Address of in-tile row `at.row0` of tile column 0 of the unit's band, per operand.
template <int ELEM>
__device__ __forceinline__ unsigned char* rms_unit_base(
        const RmsParams& p, const Operand& operand, const RmsUnit& at) {
    const uint64_t plane = operand_plane(operand, p.leading, at.index);
    return operand.base
            + (plane * operand.tile_rows + at.tr) * operand.tile_cols
                    * static_cast<uint64_t>(kTileSlots * ELEM)
            + static_cast<size_t>(at.row0) * (kTile * ELEM);
}

// Rows of more than 2048 values in the lane order: the pipelined kernel of
// rmsnorm_long.cu. Returns IOMB_OK after a launch, IOMB_ERR_UNSUPPORTED (without
// touching the error text) when the request is not one it serves.
int launch_rmsnorm_long(const RmsParams& base, uint32_t elem, bool fused, uint64_t row_bytes,
                        uint64_t bands, uint64_t x_storage_bytes, uint64_t residual_storage_bytes,
                        cudaStream_t stream, bool* launched);

}  // namespace iomb
