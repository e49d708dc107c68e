// The stages of causal grouped-query attention that are not matrix products:
// scale + causal mask, row softmax, and canonical zeros/NaNs of the merged output.
//
// Reference: src/cuda/sdpa_nonmatrix.cu:347-507 runs one thread per score (scale/mask),
// one thread per row walking its tokens four times (softmax) and one thread per output
// element (canonicalisation). Here a row group is one CTA's job: 32 rows, whose sums of
// exponentials are the 32 lanes of one warp adding in token order (the order is part of
// the result), fed through shared memory by sixteen warps that evaluate expf, so the
// additions overlap the exponentials and the global loads; every global access is a
// coalesced row segment.
//
// Workspace layout (src/cuda/sdpa_nonmatrix_request.hpp:22-49): scores FP32 and
// probability BF16, both [planes, Hq, Rp, Lp] row-major with Rp = pad16(R), Lp = pad16(L),
// so every row starts on a 64-byte (scores) / 32-byte (probability) boundary.
#include "host.hpp"

#include <math.h>

namespace iomb {

namespace {

constexpr int kGroupRows = 32;        // rows of one CTA job = lanes of the summing warp
constexpr int kChunk = 256;           // tokens of one shared-memory tile
constexpr int kExpWarps = 16;         // warps that fill the tiles (2 rows each)
constexpr int kSoftmaxWarps = kExpWarps + 1;
constexpr int kSoftmaxThreads = kSoftmaxWarps * 32;
constexpr int kSoftmaxCtasPerSm = 2;  // 17 warps each; 8 + 1 warps x 3 CTAs measured 298 against 246 us
constexpr int kScaleThreads = 256;
constexpr int kLaneRowsPerSm = 256;   // rows per SM from which one lane per row can pay
constexpr uint32_t kLaneLongestRow = 512;  // ... and only for rows this short

// Row classes of the special-value policy (src/cuda/sdpa_nonmatrix.cu:393-446).
constexpr uint32_t kRowOrdinary = 0;
constexpr uint32_t kRowNan = 1;       // a NaN among the visible scores, or only -inf
constexpr uint32_t kRowInfinite = 2;  // one or more +inf: equal shares
constexpr uint32_t kRowAbsent = 3;    // past the last logical row

struct StageParams {
    float* scores;
    uint16_t* probability;
    uint64_t rows_total;  // planes * Hq * R
    uint64_t a;
    uint32_t R, Rp, L, Lp;
    float scale;          // 1 / sqrtf(D), both correctly rounded
};

__device__ __forceinline__ float scaled_score(float score, float scale) {
    const float product = __fmul_rn(score, scale);
    return product == 0.0f ? 0.0f : product;   // a zero product is stored as +0
}

// BF16 round-to-nearest-even of src/cuda/sdpa_nonmatrix.cu:317-336: infinities kept,
// every NaN the quiet 0x7FC0, both zeros +0, subnormals rounded like normals.
__device__ __forceinline__ uint16_t probability_bits(float value) {
    const uint32_t bits = __float_as_uint(value);
    if ((bits & 0x7f800000u) == 0x7f800000u) {
        return (bits & 0x007fffffu) == 0 ? static_cast<uint16_t>(bits >> 16) : uint16_t{0x7fc0};
    }
    if ((bits & 0x7fffffffu) == 0) return 0;
    return static_cast<uint16_t>((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

__device__ __forceinline__ bool is_positive_infinity(float value) {
    return __float_as_uint(value) == 0x7f800000u;
}

__device__ __forceinline__ bool is_negative_infinity(float value) {
    return __float_as_uint(value) == 0xff800000u;
}

// Element offset of logical row `index` (plane, head, row flattened) and its visible length.
__device__ __forceinline__ void locate_row(const StageParams& p, uint64_t index,
                                           uint64_t* base, uint32_t* visible) {
    const uint64_t head = index / p.R;
    const uint32_t row = static_cast<uint32_t>(index - head * p.R);
    *base = (head * p.Rp + row) * p.Lp;
    const uint64_t causal = p.a + row + 1;
    *visible = causal < p.L ? static_cast<uint32_t>(causal) : p.L;
}

// One warp per row: 32-byte vectors over the visible prefix, the ragged end by element.
__global__ void __launch_bounds__(kScaleThreads)
scale_mask_kernel(const StageParams p) {
    constexpr int kWarps = kScaleThreads / 32;
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kWarps;
    for (uint64_t index = static_cast<uint64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
         index < p.rows_total; index += warps) {
        uint64_t base;
        uint32_t visible;
        locate_row(p, index, &base, &visible);
        float* row = p.scores + base;
        const uint32_t whole = visible & ~7u;
        for (uint32_t t = lane * 8; t < whole; t += 256) {
            uint4 lo, hi;
            load_u8_stream(row + t, &lo, &hi);
            uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                w[k] = __float_as_uint(scaled_score(__uint_as_float(w[k]), p.scale));
            }
            store_u8_stream(row + t, make_uint4(w[0], w[1], w[2], w[3]),
                            make_uint4(w[4], w[5], w[6], w[7]));
        }
        const uint32_t t = whole + lane;
        if (t < visible) row[t] = scaled_score(row[t], p.scale);
    }
}

// Row softmax. SCALE: the scores are raw and every load applies scaled_score first
// (the fused scale/mask + softmax); KEEP (with SCALE): the first pass also stores the
// scaled scores, after which the later passes read them as they are.
//
// Per group of 32 logical rows:
//   pass A  every warp takes rows w, w+17, ...: one NaN-propagating maximum per score
//           classifies the row (NaN: a NaN was seen; -inf: nothing but -inf; +inf: the
//           equal-share case, whose +inf are then counted; else the finite maximum);
//   pass B  warps 0..15 write expf(s - m) for 32 rows x 256 tokens into one of two
//           shared tiles (+0 beyond a row's visible prefix and for special rows), warp 16
//           adds the previous tile, lane r walking row r in token order: the sum of the
//           reference, which starts at +0 and skips nothing but -inf scores, whose
//           exponential is +0. Rows are 260 floats apart, so the 16-byte reads of eight
//           neighbouring lanes fall into eight different bank groups;
//   pass C  (row, 512-token segment) items over all warps, both halves loaded first: BF16_RNE(expf(s - m) / sum)
//           for the visible tokens, +0 up to L, 16-byte stores. The quotient is formed as
//           expf(s - m) * RN(1 / sum), which lies within two FP32 steps of the correctly
//           rounded quotient; unless its low half is within four steps of the BF16 tie
//           (5 codes in 8192) both round to the same BF16, and in that case the true
//           division is done instead.
constexpr int kRowStride = kChunk + 4;

__device__ __forceinline__ float max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

__device__ __forceinline__ float negative_infinity() { return __uint_as_float(0xff800000u); }

// BF16 code of a probability in [0, 1] that is not a NaN: plain round-to-nearest-even on
// the bits (a zero stays 0, subnormals round like normals).
__device__ __forceinline__ uint32_t round_bits(uint32_t bits) {
    return (bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16;
}

__device__ __forceinline__ bool near_tie(uint32_t bits) {
    return ((bits + 4u) & 0xffffu) - 0x8000u <= 8u;
}

__device__ __forceinline__ uint32_t quotient_bits(float e, float sum, float reciprocal) {
    uint32_t bits = __float_as_uint(__fmul_rn(e, reciprocal));
    if (near_tie(bits)) bits = __float_as_uint(__fdiv_rn(e, sum));
    return round_bits(bits);
}

// Eight quotients at once: the products first, without a branch between them, then the
// true division for the (rare) lanes that hold a product near a tie.
__device__ __forceinline__ void quotient_bits8(const float (&s)[8], float maximum, float sum,
                                               float reciprocal, uint32_t (&cell)[8]) {
    float e[8];
    uint32_t bits[8];
    bool risky = false;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        e[k] = expf(__fsub_rn(s[k], maximum));
        bits[k] = __float_as_uint(__fmul_rn(e[k], reciprocal));
        risky |= near_tie(bits[k]);
    }
    if (risky) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (near_tie(bits[k])) bits[k] = __float_as_uint(__fdiv_rn(e[k], sum));
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) cell[k] = round_bits(bits[k]);
}

template <bool SCALE, bool KEEP>
__global__ void __launch_bounds__(kSoftmaxThreads, kSoftmaxCtasPerSm)
softmax_kernel(const StageParams p) {
    extern __shared__ __align__(16) float tile[];   // [2][kGroupRows][kRowStride]
    __shared__ uint64_t s_base[kGroupRows];
    __shared__ uint32_t s_visible[kGroupRows];
    __shared__ uint32_t s_class[kGroupRows];
    __shared__ float s_max[kGroupRows];
    __shared__ float s_sum[kGroupRows];    // the sum, or 1 / count for a +inf row
    __shared__ uint32_t s_chunks;

    constexpr bool kScaleLater = SCALE && !KEEP;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = threadIdx.x >> 5;
    const uint64_t groups = (p.rows_total + kGroupRows - 1) / kGroupRows;
    const uint32_t segments = (p.L + 511u) / 512u;

    for (uint64_t group = blockIdx.x; group < groups; group += gridDim.x) {
        __syncthreads();   // the previous group's readers are done with the row records
        if (threadIdx.x < kGroupRows) {
            const uint64_t index = group * kGroupRows + threadIdx.x;
            uint64_t base = 0;
            uint32_t visible = 0;
            if (index < p.rows_total) locate_row(p, index, &base, &visible);
            s_base[threadIdx.x] = base;
            s_visible[threadIdx.x] = visible;
        }
        __syncthreads();

        // ---- pass A ---------------------------------------------------------------
        for (uint32_t r = warp; r < kGroupRows; r += kSoftmaxWarps) {
            const uint32_t visible = s_visible[r];
            if (visible == 0) {
                if (lane == 0) s_class[r] = kRowAbsent;
                continue;
            }
            float* row = p.scores + s_base[r];
            float top = negative_infinity();
            for (uint32_t t0 = lane * 4; t0 < visible; t0 += 4 * 128) {
                float4 v[4];                      // four row segments in flight per lane
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t t = t0 + u * 128;
                    if (t < visible) v[u] = *reinterpret_cast<const float4*>(row + t);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t t = t0 + u * 128;
                    if (t >= visible) break;
                    float s[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                    if constexpr (SCALE) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) s[k] = scaled_score(s[k], p.scale);
                    }
                    if (t + 4 <= visible) {
                        top = max_nan(max_nan(max_nan(top, s[0]), max_nan(s[1], s[2])), s[3]);
                        if constexpr (KEEP) {
                            *reinterpret_cast<float4*>(row + t) = make_float4(s[0], s[1], s[2], s[3]);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (t + k >= visible) continue;
                            top = max_nan(top, s[k]);
                            if constexpr (KEEP) row[t + k] = s[k];
                        }
                    }
                }
            }
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) {
                top = max_nan(top, __shfl_xor_sync(0xffffffffu, top, offset));
            }
            uint32_t positive = 0;
            if constexpr (KEEP) __syncwarp();   // the scaled scores of the other lanes
            if (is_positive_infinity(top)) {   // rare: count the +inf scores of the row
                for (uint32_t t = lane; t < visible; t += 32) {
                    float s = row[t];
                    if constexpr (kScaleLater) s = scaled_score(s, p.scale);
                    positive += is_positive_infinity(s) ? 1u : 0u;
                }
#pragma unroll
                for (int offset = 16; offset > 0; offset >>= 1) {
                    positive += __shfl_xor_sync(0xffffffffu, positive, offset);
                }
            }
            if (lane == 0) {
                if (top != top || is_negative_infinity(top)) {
                    s_class[r] = kRowNan;
                } else if (positive != 0) {
                    s_class[r] = kRowInfinite;
                    s_sum[r] = __fdiv_rn(1.0f, static_cast<float>(positive));
                } else {
                    s_class[r] = kRowOrdinary;
                    s_max[r] = top;
                }
            }
        }
        __syncthreads();
        if (warp == 0) {
            uint32_t longest = s_class[lane] == kRowOrdinary ? s_visible[lane] : 0u;
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) {
                longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, offset));
            }
            if (lane == 0) s_chunks = (longest + kChunk - 1) / kChunk;
        }
        __syncthreads();
        // ---- pass B ---------------------------------------------------------------
        const uint32_t chunks = s_chunks;
        float running = 0.0f;
        for (uint32_t c = 0; c <= chunks; ++c) {
            if (warp < kExpWarps && c < chunks) {
                float* buffer = tile + (c & 1u) * (kGroupRows * kRowStride);
                constexpr uint32_t kRowsPerWarp = kGroupRows / kExpWarps;
                constexpr uint32_t kVectors = kChunk / 128;      // float4 per lane and row
                float4 v[kRowsPerWarp][kVectors];
#pragma unroll
                for (uint32_t rr = 0; rr < kRowsPerWarp; ++rr) {
                    const uint32_t r = warp * kRowsPerWarp + rr;
                    const uint32_t visible = s_class[r] == kRowOrdinary ? s_visible[r] : 0u;
                    const float* row = p.scores + s_base[r];
#pragma unroll
                    for (uint32_t k = 0; k < kVectors; ++k) {
                        const uint32_t t = c * kChunk + k * 128 + lane * 4;
                        v[rr][k] = t < visible ? *reinterpret_cast<const float4*>(row + t)
                                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
                }
#pragma unroll
                for (uint32_t rr = 0; rr < kRowsPerWarp; ++rr) {
                    const uint32_t r = warp * kRowsPerWarp + rr;
                    const uint32_t visible = s_class[r] == kRowOrdinary ? s_visible[r] : 0u;
                    const float maximum = s_max[r];
#pragma unroll
                    for (uint32_t k = 0; k < kVectors; ++k) {
                        const uint32_t t = c * kChunk + k * 128 + lane * 4;
                        float s[4] = {v[rr][k].x, v[rr][k].y, v[rr][k].z, v[rr][k].w};
                        float e[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (t + 4 <= visible) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if constexpr (kScaleLater) s[j] = scaled_score(s[j], p.scale);
                                e[j] = expf(__fsub_rn(s[j], maximum));
                            }
                        } else if (t < visible) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (t + j >= visible) continue;
                                if constexpr (kScaleLater) s[j] = scaled_score(s[j], p.scale);
                                e[j] = expf(__fsub_rn(s[j], maximum));
                            }
                        }
                        *reinterpret_cast<float4*>(buffer + r * kRowStride + k * 128 + lane * 4) =
                                make_float4(e[0], e[1], e[2], e[3]);
                    }
                }
            } else if (warp == kExpWarps && c > 0) {
                const float4* column = reinterpret_cast<const float4*>(
                        tile + ((c - 1) & 1u) * (kGroupRows * kRowStride) + lane * kRowStride);
#pragma unroll 8
                for (uint32_t t = 0; t < kChunk / 4; ++t) {
                    const float4 e = column[t];
                    running = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(running, e.x), e.y), e.z), e.w);
                }
            }
            __syncthreads();
        }
        if (warp == kExpWarps && s_class[lane] == kRowOrdinary) s_sum[lane] = running;
        __syncthreads();

        // ---- pass C ---------------------------------------------------------------
        for (uint32_t item = warp; item < kGroupRows * segments; item += kSoftmaxWarps) {
            const uint32_t r = item / segments;
            const uint32_t row_class = s_class[r];
            if (row_class == kRowAbsent) continue;
            const uint32_t t0 = (item - r * segments) * 512u + lane * 8;
            const uint32_t visible = s_visible[r];
            const float* row = p.scores + s_base[r];
            uint16_t* out = p.probability + s_base[r];
            const float sum = s_sum[r];
            const float maximum = s_max[r];
            float4 lo[2], hi[2];                  // both halves of the segment in flight
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const uint32_t t = t0 + u * 256;
                if (t < visible && row_class != kRowNan) {
                    lo[u] = *reinterpret_cast<const float4*>(row + t);
                    hi[u] = *reinterpret_cast<const float4*>(row + t + 4);
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const uint32_t t = t0 + u * 256;
                if (t >= p.L) break;
                uint32_t cell[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (t < visible) {
                    if (row_class == kRowNan) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) cell[k] = t + k < visible ? 0x7fc0u : 0u;
                    } else {
                        float s[8] = {lo[u].x, lo[u].y, lo[u].z, lo[u].w, hi[u].x, hi[u].y, hi[u].z, hi[u].w};
                        if constexpr (kScaleLater) {
#pragma unroll
                            for (int k = 0; k < 8; ++k) s[k] = scaled_score(s[k], p.scale);
                        }
                        if (row_class == kRowInfinite) {
                            const uint32_t share = probability_bits(sum);
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                cell[k] = t + k < visible && is_positive_infinity(s[k]) ? share : 0u;
                            }
                        } else {
                            const float reciprocal = __frcp_rn(sum);
                            if (t + 8 <= visible) {
                                quotient_bits8(s, maximum, sum, reciprocal, cell);
                            } else {
#pragma unroll
                                for (int k = 0; k < 8; ++k) {
                                    if (t + k >= visible) continue;
                                    cell[k] = quotient_bits(expf(__fsub_rn(s[k], maximum)), sum, reciprocal);
                                }
                            }
                        }
                    }
                }
                if (t + 8 <= p.L) {
                    *reinterpret_cast<uint4*>(out + t) = make_uint4(
                            cell[0] | (cell[1] << 16), cell[2] | (cell[3] << 16),
                            cell[4] | (cell[5] << 16), cell[6] | (cell[7] << 16));
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        if (t + k < p.L) out[t + k] = static_cast<uint16_t>(cell[k]);
                    }
                }
            }
        }
    }
}

// Row softmax with one LANE per row, for requests with many short rows. A lane walks its own row three times (maximum, sum in token order, probabilities)
// with four 32-byte loads in flight, so the additions of 32 rows run side by side in one warp
// and nothing waits at a barrier. Slots are ordered longest prefix first and head-minor: the
// lanes of a warp hold the same query row of 32 different heads, hence the same prefix
// length, and the long rows start first. Each lane reads whole 128-byte lines of its row
// per batch; its 16-byte probability stores meet in L2.
constexpr int kLaneThreads = 64;
constexpr int kLaneBatch = 4;          // 32-byte vectors per lane in flight

__device__ __forceinline__ void load_f8(const float* address, float (&v)[8]) {
    asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]),
                   "=f"(v[6]), "=f"(v[7])
                 : "l"(address));
}

__device__ __forceinline__ void store_f8(float* address, const float (&v)[8]) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(address), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]),
                    "f"(v[6]), "f"(v[7])
                 : "memory");
}

template <bool SCALE, bool KEEP>
__global__ void __launch_bounds__(kLaneThreads)
softmax_rows_kernel(const StageParams p) {
    constexpr bool kScaleLater = SCALE && !KEEP;
    const uint64_t slot = static_cast<uint64_t>(blockIdx.x) * kLaneThreads + threadIdx.x;
    if (slot >= p.rows_total) return;
    const uint64_t heads = p.rows_total / p.R;
    const uint64_t step = slot / heads;
    const uint64_t head = slot - step * heads;
    const uint32_t row_index = p.R - 1 - static_cast<uint32_t>(step);
    float* row = p.scores + (head * p.Rp + row_index) * p.Lp;
    uint16_t* out = p.probability + (head * p.Rp + row_index) * p.Lp;
    const uint64_t causal = p.a + row_index + 1;
    const uint32_t visible = causal < p.L ? static_cast<uint32_t>(causal) : p.L;

    // ---- pass A: NaN-propagating maximum --------------------------------------------
    float top = negative_infinity();
    for (uint32_t t0 = 0; t0 < visible; t0 += 8 * kLaneBatch) {
        float v[kLaneBatch][8];
#pragma unroll
        for (int u = 0; u < kLaneBatch; ++u) {
            if (t0 + u * 8 < visible) load_f8(row + t0 + u * 8, v[u]);
        }
#pragma unroll
        for (int u = 0; u < kLaneBatch; ++u) {
            const uint32_t t = t0 + u * 8;
            if (t >= visible) break;
            if constexpr (SCALE) {
#pragma unroll
                for (int k = 0; k < 8; ++k) v[u][k] = scaled_score(v[u][k], p.scale);
            }
            if (t + 8 <= visible) {
                top = max_nan(top, max_nan(max_nan(max_nan(v[u][0], v[u][1]), max_nan(v[u][2], v[u][3])),
                                           max_nan(max_nan(v[u][4], v[u][5]), max_nan(v[u][6], v[u][7]))));
                if constexpr (KEEP) store_f8(row + t, v[u]);
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (t + k >= visible) continue;
                    top = max_nan(top, v[u][k]);
                    if constexpr (KEEP) row[t + k] = v[u][k];
                }
            }
        }
    }
    uint32_t row_class = kRowOrdinary;
    float sum = 0.0f;
    if (top != top || is_negative_infinity(top)) {
        row_class = kRowNan;
    } else if (is_positive_infinity(top)) {
        uint32_t positive = 0;
        for (uint32_t t = 0; t < visible; ++t) {
            float s = row[t];
            if constexpr (kScaleLater) s = scaled_score(s, p.scale);
            positive += is_positive_infinity(s) ? 1u : 0u;
        }
        row_class = kRowInfinite;
        sum = __fdiv_rn(1.0f, static_cast<float>(positive));
    }

    // ---- pass B: the sum, in token order ------------------------------------------
    if (row_class == kRowOrdinary) {
        for (uint32_t t0 = 0; t0 < visible; t0 += 8 * kLaneBatch) {
            float v[kLaneBatch][8];
#pragma unroll
            for (int u = 0; u < kLaneBatch; ++u) {
                if (t0 + u * 8 < visible) load_f8(row + t0 + u * 8, v[u]);
            }
#pragma unroll
            for (int u = 0; u < kLaneBatch; ++u) {
                const uint32_t t = t0 + u * 8;
                if (t >= visible) break;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if constexpr (kScaleLater) v[u][k] = scaled_score(v[u][k], p.scale);
                    v[u][k] = expf(__fsub_rn(v[u][k], top));
                }
                if (t + 8 <= visible) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) sum = __fadd_rn(sum, v[u][k]);
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        if (t + k < visible) sum = __fadd_rn(sum, v[u][k]);
                    }
                }
            }
        }
    }

    // ---- pass C: probabilities -----------------------------------------------------
    const float reciprocal = __frcp_rn(sum);
    const uint32_t share = probability_bits(sum);
    for (uint32_t t0 = 0; t0 < p.L; t0 += 8 * kLaneBatch) {
        float v[kLaneBatch][8];
#pragma unroll
        for (int u = 0; u < kLaneBatch; ++u) {
            if (t0 + u * 8 < visible && row_class != kRowNan) load_f8(row + t0 + u * 8, v[u]);
        }
#pragma unroll
        for (int u = 0; u < kLaneBatch; ++u) {
            const uint32_t t = t0 + u * 8;
            if (t >= p.L) break;
            uint32_t cell[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (t < visible) {
                if (row_class == kRowNan) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) cell[k] = t + k < visible ? 0x7fc0u : 0u;
                } else {
                    if constexpr (kScaleLater) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) v[u][k] = scaled_score(v[u][k], p.scale);
                    }
                    if (row_class == kRowInfinite) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            cell[k] = t + k < visible && is_positive_infinity(v[u][k]) ? share : 0u;
                        }
                    } else if (t + 8 <= visible) {
                        quotient_bits8(v[u], top, sum, reciprocal, cell);
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            if (t + k >= visible) continue;
                            cell[k] = quotient_bits(expf(__fsub_rn(v[u][k], top)), sum, reciprocal);
                        }
                    }
                }
            }
            if (t + 8 <= p.L) {
                *reinterpret_cast<uint4*>(out + t) = make_uint4(
                        cell[0] | (cell[1] << 16), cell[2] | (cell[3] << 16),
                        cell[4] | (cell[5] << 16), cell[6] | (cell[7] << 16));
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (t + k < p.L) out[t + k] = static_cast<uint16_t>(cell[k]);
                }
            }
        }
    }
}

// Canonical zeros and NaNs of a BF16 view: one warp per 16x16 tile (32 lanes x 16 bytes),
// four tiles per warp, the store issued only where a value changed.
constexpr int kCanonThreads = 256;
constexpr uint32_t kCanonTiles = 4;
constexpr int kCanonUnroll = 4;

struct CanonParams {
    Operand out;
    Leading leading;
    uint64_t items;       // planes * tile_rows * ceil(tile_cols / kCanonTiles)
    uint32_t rows, cols, tile_rows, tile_cols, groups;
};

__device__ __forceinline__ uint32_t canonical_pair(uint32_t word) {
    uint32_t lo = word & 0xffffu, hi = word >> 16;
    if ((lo & 0x7fffu) == 0) lo = 0;
    else if ((lo & 0x7f80u) == 0x7f80u && (lo & 0x007fu) != 0) lo = 0x7fc0u;
    if ((hi & 0x7fffu) == 0) hi = 0;
    else if ((hi & 0x7f80u) == 0x7f80u && (hi & 0x007fu) != 0) hi = 0x7fc0u;
    return lo | (hi << 16);
}

// Non-zero when one of the word's two BF16 codes may need rewriting: an all-ones exponent
// (infinity or NaN) or a zero magnitude with the sign set. Seven logic / add operations per
// word; the exact rule (canonical_pair) then runs only on words that are flagged.
__device__ __forceinline__ uint32_t suspicious_pair(uint32_t word) {
    // 0x7f80 + 0x0080 reaches bit 15 exactly for an all-ones exponent (no carry across halves)
    const uint32_t special = ((word & 0x7f807f80u) + 0x00800080u) & 0x80008000u;
    // a magnitude m <= 0x7fff plus 0x7fff reaches bit 15 exactly when m != 0
    const uint32_t nonzero = ((word & 0x7fff7fffu) + 0x7fff7fffu) & 0x80008000u;
    return special | (word & ~nonzero & 0x80008000u);
}

__global__ void __launch_bounds__(kCanonThreads)
canonicalize_kernel(const CanonParams p) {
    constexpr int kWarps = kCanonThreads / 32;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = lane >> 1, col = (lane & 1u) * 8;
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kWarps;
    for (uint64_t item = static_cast<uint64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
         item < p.items; item += warps) {
        const uint32_t g = static_cast<uint32_t>(item % p.groups);
        const uint64_t band = item / p.groups;
        const uint32_t tr = static_cast<uint32_t>(band % p.tile_rows);
        const uint64_t index = band / p.tile_rows;
        if (row >= p.rows - tr * kTile) continue;
        unsigned char* first = p.out.base
                + ((operand_plane(p.out, p.leading, index) * p.tile_rows + tr) * p.tile_cols) * 512ull
                + lane * 16;
        const uint32_t tc0 = g * kCanonTiles;
        uint4 value[kCanonTiles];
        uint32_t valid[kCanonTiles];
#pragma unroll
        for (uint32_t k = 0; k < kCanonTiles; ++k) {
            const uint32_t tc = tc0 + k;
            valid[k] = 0;
            if (tc < p.tile_cols) {
                const uint32_t cols_left = p.cols - tc * kTile;
                valid[k] = col < cols_left ? min(8u, cols_left - col) : 0u;
            }
            if (valid[k] != 0) value[k] = load_u4(first + (tc0 + k) * 512ull);
        }
#pragma unroll
        for (uint32_t k = 0; k < kCanonTiles; ++k) {
            if (valid[k] == 0) continue;
            unsigned char* address = first + (tc0 + k) * 512ull;
            if ((suspicious_pair(value[k].x) | suspicious_pair(value[k].y) | suspicious_pair(value[k].z)
                 | suspicious_pair(value[k].w)) == 0) {
                continue;
            }
            const uint4 clean = make_uint4(canonical_pair(value[k].x), canonical_pair(value[k].y),
                                           canonical_pair(value[k].z), canonical_pair(value[k].w));
            if (valid[k] == 8) {
                if (clean.x != value[k].x || clean.y != value[k].y || clean.z != value[k].z
                    || clean.w != value[k].w) {
                    store_u4(address, clean);
                }
            } else {
                const uint32_t words[4] = {clean.x, clean.y, clean.z, clean.w};
                uint16_t* cells = reinterpret_cast<uint16_t*>(address);
                for (uint32_t e = 0; e < valid[k]; ++e) {
                    cells[e] = static_cast<uint16_t>(words[e >> 1] >> ((e & 1u) * 16));
                }
            }
        }
    }
}

// The same over a dense run of whole tiles (contiguous planes, both extents multiples of
// 16): 32-byte loads, four per thread in flight, one-shot grid (a persistent grid with
// eight loads in flight measured 3.2 against 4.0 TB/s).
__global__ void __launch_bounds__(kCanonThreads)
canonicalize_linear_kernel(unsigned char* data, uint64_t pairs) {
    constexpr int kUnroll = kCanonUnroll;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kCanonThreads;
    for (uint64_t first = static_cast<uint64_t>(blockIdx.x) * kCanonThreads * kUnroll + threadIdx.x;
         first < pairs; first += stride * kUnroll) {
        uint4 lo[kUnroll], hi[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint64_t i = first + static_cast<uint64_t>(u) * kCanonThreads;
            if (i < pairs) load_u8_stream(data + i * 32, &lo[u], &hi[u]);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint64_t i = first + static_cast<uint64_t>(u) * kCanonThreads;
            if (i >= pairs) break;
            if ((suspicious_pair(lo[u].x) | suspicious_pair(lo[u].y) | suspicious_pair(lo[u].z)
                 | suspicious_pair(lo[u].w) | suspicious_pair(hi[u].x) | suspicious_pair(hi[u].y)
                 | suspicious_pair(hi[u].z) | suspicious_pair(hi[u].w)) == 0) {
                continue;
            }
            const uint4 a = make_uint4(canonical_pair(lo[u].x), canonical_pair(lo[u].y),
                                       canonical_pair(lo[u].z), canonical_pair(lo[u].w));
            const uint4 b = make_uint4(canonical_pair(hi[u].x), canonical_pair(hi[u].y),
                                       canonical_pair(hi[u].z), canonical_pair(hi[u].w));
            const uint32_t changed = (a.x ^ lo[u].x) | (a.y ^ lo[u].y) | (a.z ^ lo[u].z) | (a.w ^ lo[u].w)
                    | (b.x ^ hi[u].x) | (b.y ^ hi[u].y) | (b.z ^ hi[u].z) | (b.w ^ hi[u].w);
            if (changed != 0) store_u8_stream(data + i * 32, a, b);
        }
    }
}

// ---- admission ------------------------------------------------------------------

bool mul_overflows(uint64_t a, uint64_t b, uint64_t* out) {
    return __builtin_mul_overflow(a, b, out);
}

// The rules of validate_geometry / validate_sdpa_nonmatrix_request
// (src/cuda/sdpa_nonmatrix.cu:82-229,509-562) for the two workspace segments.
int check_stages(const iomb_sdpa_stages* stages, const char* what, StageParams* p) {
    if (stages == nullptr) return fail(IOMB_ERR_INVALID_ARGUMENT, "sdpa stages: null request");
    const iomb_sdpa_stages& q = *stages;
    if (q.scores == nullptr || q.probability == nullptr) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "sdpa stages: workspace pointers must be non-null");
    }
    if (q.Hq == 0 || q.Hkv == 0 || q.R == 0 || q.C == 0 || q.D == 0 || q.L == 0 || q.planes == 0) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "sdpa stages: dimensions must be nonzero");
    }
    if (q.L > q.C || q.a >= q.C || q.R > q.C - q.a) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "sdpa stages: causal dimensions are invalid");
    }
    if (q.Hq % q.Hkv != 0) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "sdpa stages: Hq is not a multiple of Hkv");
    }
    if (q.R > 0x7fffffffull || q.L > 0x7fffffffull || q.D > (1ull << 24)) {
        return fail(IOMB_ERR_UNSUPPORTED, "sdpa stages: extent exceeds the kernel limit");
    }
    const uint64_t Rp = (q.R + 15) / 16 * 16, Lp = (q.L + 15) / 16 * 16;
    uint64_t heads = 0, rows = 0, cells = 0, score_bytes = 0, logical_rows = 0;
    if (mul_overflows(q.planes, q.Hq, &heads) || mul_overflows(heads, Rp, &rows)
        || mul_overflows(rows, Lp, &cells) || mul_overflows(cells, 4, &score_bytes)
        || mul_overflows(heads, q.R, &logical_rows)) {
        return fail(IOMB_ERR_OVERFLOW, "sdpa stages: score extent overflows");
    }
    const uintptr_t s0 = reinterpret_cast<uintptr_t>(q.scores);
    const uintptr_t p0 = reinterpret_cast<uintptr_t>(q.probability);
    if ((s0 & 31u) != 0 || (p0 & 31u) != 0) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "sdpa stages: workspace segments must be 32-byte aligned");
    }
    if (s0 + score_bytes < s0 || p0 + cells * 2 < p0) {
        return fail(IOMB_ERR_OVERFLOW, "sdpa stages: pointer range overflows");
    }
    if (s0 < p0 + cells * 2 && p0 < s0 + score_bytes) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "sdpa stages: scores and probability ranges overlap");
    }
    (void)what;
    p->scores = q.scores;
    p->probability = static_cast<uint16_t*>(q.probability);
    p->rows_total = logical_rows;
    p->a = q.a;
    p->R = static_cast<uint32_t>(q.R);
    p->Rp = static_cast<uint32_t>(Rp);
    p->L = static_cast<uint32_t>(q.L);
    p->Lp = static_cast<uint32_t>(Lp);
    p->scale = 1.0f / sqrtf(static_cast<float>(q.D));
    return IOMB_OK;
}

int softmax_launch(const iomb_sdpa_stages* stages, bool scale, bool keep, void* stream) {
    StageParams p{};
    const int status = check_stages(stages, "sdpa softmax", &p);
    if (status != IOMB_OK) return status;
    if (sm_count() <= 0) return fail(IOMB_ERR_DEVICE, "sdpa softmax: no CUDA device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // One lane per row pays when every SM gets at least kLaneRowsPerSm rows and the rows are
    // short: each lane then fetches its own 128-byte lines, which costs DRAM page locality
    // that grows with the row length (L 512, 131 072 rows: 159 us against 194 us grouped;
    // L 2048, 65 536 rows: 1218 us against 315 us).
    if (p.L <= kLaneLongestRow && p.rows_total >= static_cast<uint64_t>(kLaneRowsPerSm) * sm_count()) {
        auto rows_kernel = !scale ? softmax_rows_kernel<false, false>
                                  : (keep ? softmax_rows_kernel<true, true> : softmax_rows_kernel<true, false>);
        const uint64_t ctas = (p.rows_total + kLaneThreads - 1) / kLaneThreads;
        if (ctas > 0x7fffffffull) return fail(IOMB_ERR_UNSUPPORTED, "sdpa softmax: too many rows");
        rows_kernel<<<static_cast<unsigned>(ctas), kLaneThreads, 0, s>>>(p);
        return check_launch("sdpa softmax launch");
    }
    const unsigned grid = grid_for((p.rows_total + kGroupRows - 1) / kGroupRows, kSoftmaxCtasPerSm);
    constexpr int kTileBytes = 2 * kGroupRows * kRowStride * static_cast<int>(sizeof(float));
    auto kernel = !scale ? softmax_kernel<false, false>
                         : (keep ? softmax_kernel<true, true> : softmax_kernel<true, false>);
    const int prepared = allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
    if (prepared != IOMB_OK) return prepared;
    kernel<<<grid, kSoftmaxThreads, kTileBytes, s>>>(p);
    return check_launch("sdpa softmax launch");
}

}  // namespace

int prepare_sdpa_kernels() {
    const void* kernels[3] = {reinterpret_cast<const void*>(softmax_kernel<false, false>),
                              reinterpret_cast<const void*>(softmax_kernel<true, true>),
                              reinterpret_cast<const void*>(softmax_kernel<true, false>)};
    for (const void* kernel : kernels) {
        const int status = allow_full_shared_memory(kernel);
        if (status != IOMB_OK) return status;
    }
    return IOMB_OK;
}

}  // namespace iomb

extern "C" int iomb_sdpa_scale_mask(const iomb_sdpa_stages* stages, void* stream) {
    iomb::StageParams p{};
    const int status = iomb::check_stages(stages, "sdpa scale_mask", &p);
    if (status != IOMB_OK) return status;
    if (iomb::sm_count() <= 0) return iomb::fail(IOMB_ERR_DEVICE, "sdpa scale_mask: no CUDA device");
    const uint64_t ctas = (p.rows_total + iomb::kScaleThreads / 32 - 1) / (iomb::kScaleThreads / 32);
    iomb::scale_mask_kernel<<<iomb::grid_one_shot(ctas), iomb::kScaleThreads, 0,
                              static_cast<cudaStream_t>(stream)>>>(p);
    return iomb::check_launch("sdpa scale_mask launch");
}

extern "C" int iomb_sdpa_softmax(const iomb_sdpa_stages* stages, void* stream) {
    return iomb::softmax_launch(stages, false, false, stream);
}

extern "C" int iomb_sdpa_scale_mask_softmax(const iomb_sdpa_stages* stages, int keep_scores,
                                            void* stream) {
    return iomb::softmax_launch(stages, true, keep_scores != 0, stream);
}

extern "C" int iomb_sdpa_canonicalize_output(const iomb_view* out, void* stream) {
    using namespace iomb;
    ViewFacts facts{};
    const int status = check_view(out, "sdpa output", &facts);
    if (status != IOMB_OK) return status;
    if (out->dtype != IOMB_BF16) return fail(IOMB_ERR_UNSUPPORTED, "sdpa output: leaf is not BF16");
    if (facts.rows > 0xFFFFFFFFull || facts.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "sdpa output: matrix extent exceeds the kernel limit");
    }
    if (sm_count() <= 0) return fail(IOMB_ERR_DEVICE, "sdpa output: no CUDA device");
    CanonParams p{};
    uint64_t strides[1][kMaxLead] = {};
    for (uint32_t axis = 0; axis < facts.leading; ++axis) strides[0][axis] = out->plane_strides[axis];
    collapse_leading(facts.leading, out->dims, strides, 1, &p.leading);
    p.out = make_operand(*out, facts, strides[0], p.leading, false, false);
    p.rows = static_cast<uint32_t>(facts.rows);
    p.cols = static_cast<uint32_t>(facts.cols);
    p.tile_rows = static_cast<uint32_t>(facts.tile_rows);
    p.tile_cols = static_cast<uint32_t>(facts.tile_cols);
    p.groups = (p.tile_cols + kCanonTiles - 1) / kCanonTiles;
    p.items = p.leading.planes * facts.tile_rows * p.groups;
    if (p.leading.contiguous && facts.rows % kTile == 0 && facts.cols % kTile == 0) {
        unsigned char* start = static_cast<unsigned char*>(out->base) + out->plane_offset * facts.plane_bytes;
        const uint64_t pairs = p.leading.planes * facts.plane_bytes / 32;
        const uint64_t per_cta = static_cast<uint64_t>(kCanonThreads) * kCanonUnroll;
        canonicalize_linear_kernel<<<grid_one_shot((pairs + per_cta - 1) / per_cta), kCanonThreads, 0,
                                     static_cast<cudaStream_t>(stream)>>>(start, pairs);
        return check_launch("sdpa canonicalize launch");
    }
    const uint64_t ctas = (p.items + kCanonThreads / 32 - 1) / (kCanonThreads / 32);
    canonicalize_kernel<<<grid_one_shot(ctas), kCanonThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("sdpa canonicalize launch");
}
