// Elementwise ADD / MUL / SUB / DIV with right-aligned broadcasting on tiled storage.
//
// Replaces grid_stride_binary_kernel / alias_safe_binary_kernel of the
// reference (src/shared/standard_tiled_add.inl:206-464). Three kernels:
//
//   binary_stream_bc_kernel  one dense full-shape operand against a single [1,N]
//                         or [M,1] plane (bias add, per-row scale): the big
//                         operand is a linear stream, the small one comes from L1.
//   binary_linear_kernel  every operand has the result's shape, tile-multiple
//                         extents and dense planes: the three storages are
//                         walked as one linear stream of 16-byte vectors.
//   binary_tiled_kernel   everything else: a warp owns a run of tiles of one
//                         16-row band; broadcast operands are fetched once per
//                         tile (row vector) or once per band (column scalar),
//                         logical bounds mask the stores so padding is never
//                         written.
//
// Arithmetic: one IEEE binary32 operation without contraction (division correctly
// rounded), one RNE encode for BF16, canonical positive quiet NaN
// (src/shared/scalar_binary_codec.hpp:120-178). Integers wrap and have no division
// (src/device_ops_binary.cpp:46-57). Each lane reads its inputs before it stores the same slots, so
// the exact in-place alias the reference handles with a shared-memory snapshot
// needs no special path here.
#include "host.hpp"

#include <type_traits>

#include <cuda_fp16.h>

namespace iomb {

enum class Leaf : int { I32 = 0, F32 = 1, BF16 = 2 };

// One IEEE binary32 operation, rounded once (never contracted); division is the
// correctly rounded quotient.
template <int OP>
__device__ __forceinline__ float apply_f32(float x, float y) {
    if constexpr (OP == IOMB_ADD) return __fadd_rn(x, y);
    if constexpr (OP == IOMB_MUL) return __fmul_rn(x, y);
    if constexpr (OP == IOMB_SUB) return __fsub_rn(x, y);
    return __fdiv_rn(x, y);
}

template <Leaf L, int OP>
__device__ __forceinline__ uint32_t apply_word(uint32_t a, uint32_t b) {
    if constexpr (L == Leaf::I32) {
        // Integers wrap; the reference admits no integer division.
        return OP == IOMB_ADD ? a + b : OP == IOMB_MUL ? a * b : a - b;
    } else if constexpr (L == Leaf::F32) {
        return f32_canonical_bits(apply_f32<OP>(__uint_as_float(a), __uint_as_float(b)));
    } else {
        if constexpr (OP == IOMB_ADD) return add_bf16x2_canonical(a, b);
        if constexpr (OP == IOMB_SUB) return sub_bf16x2_canonical(a, b);
        if constexpr (OP == IOMB_MUL) return mul_bf16x2_canonical(a, b);
        return pack_bf16x2_canonical(apply_f32<OP>(bf16_lo(a), bf16_lo(b)),
                                     apply_f32<OP>(bf16_hi(a), bf16_hi(b)));
    }
}

template <Leaf L, int OP>
__device__ __forceinline__ uint4 apply_vector(uint4 a, uint4 b) {
    return make_uint4(apply_word<L, OP>(a.x, b.x), apply_word<L, OP>(a.y, b.y),
                      apply_word<L, OP>(a.z, b.z), apply_word<L, OP>(a.w, b.w));
}

// ---- linear stream --------------------------------------------------------

constexpr int kLinearThreads = 256;
constexpr int kLinearUnroll = 4;

// One CTA streams one contiguous chunk of kLinearThreads * kLinearUnroll
// vectors per operand (16 KiB). Measured on B200, one chunk per CTA in launch
// order sustains about 13 % more HBM bandwidth than persistent grid-stride
// CTAs, so the grid covers the whole stream.
template <Leaf L, int OP>
__global__ void __launch_bounds__(kLinearThreads)
binary_linear_kernel(const uint4* lhs, const uint4* rhs, uint4* out, uint64_t vectors) {
    constexpr uint64_t kChunk = static_cast<uint64_t>(kLinearThreads) * kLinearUnroll;
    const uint64_t chunks = (vectors + kChunk - 1) / kChunk;
    for (uint64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
        const uint64_t base = chunk * kChunk + threadIdx.x;
        uint4 a[kLinearUnroll], b[kLinearUnroll];
        if (base + kLinearThreads * (kLinearUnroll - 1) < vectors) {
            // A whole chunk: each thread moves pairs of neighbouring vectors with
            // 256-bit accesses (streams start on tile boundaries, so pairs are
            // 32-byte aligned), half the load/store instructions of the 128-bit form.
            const uint64_t pair = (chunk * kChunk) / 2 + threadIdx.x;
#pragma unroll
            for (int u = 0; u < kLinearUnroll / 2; ++u) {
                const uint64_t at = 2 * (pair + u * kLinearThreads);
                load_u8_stream(lhs + at, &a[2 * u], &a[2 * u + 1]);
                load_u8_stream(rhs + at, &b[2 * u], &b[2 * u + 1]);
            }
#pragma unroll
            for (int u = 0; u < kLinearUnroll / 2; ++u) {
                const uint64_t at = 2 * (pair + u * kLinearThreads);
                store_u8_stream(out + at, apply_vector<L, OP>(a[2 * u], b[2 * u]),
                                apply_vector<L, OP>(a[2 * u + 1], b[2 * u + 1]));
            }
        } else {
            for (int u = 0; u < kLinearUnroll; ++u) {
                const uint64_t index = base + u * kLinearThreads;
                if (index < vectors) {
                    store_u4_stream(out + index,
                                    apply_vector<L, OP>(load_u4_stream(lhs + index),
                                                        load_u4_stream(rhs + index)));
                }
            }
        }
    }
}

// ---- linear stream against one broadcast row / column --------------------------
//
// `big` has the result's shape (dense planes, tile-multiple extents) and is
// streamed exactly like binary_linear_kernel; `small` is a single [1,N] or [M,1]
// plane that every leading index shares. For vector i of the stream the tile is
// i / (vectors per tile); a [1,N] operand contributes row 0 of tile column
// (tile % tile_cols), an [M,1] operand column 0 of band (tile / tile_cols) %
// tile_rows. The small operand stays in L1/L2; HBM sees the big stream only.
struct StreamBcParams {
    const uint4* big;
    const unsigned char* small;
    uint4* out;
    uint64_t vectors;
    uint32_t tile_rows;
    uint32_t tile_cols;
    uint32_t cols_shift;    // log2(tile_cols) when it is a power of two, else 32
    uint32_t single_plane;  // the stream is one plane: band index needs no modulo
};

template <Leaf L, int OP, bool COLUMN, bool SMALL_IS_LHS>
__global__ void __launch_bounds__(kLinearThreads)
binary_stream_bc_kernel(const StreamBcParams p) {
    constexpr int ELEM = L == Leaf::BF16 ? 2 : 4;
    constexpr uint32_t kTileVectors = kTileSlots * ELEM / 16;     // 32 or 64
    constexpr uint32_t kVectorsPerRow = kTile * ELEM / 16;        // 2 or 4
    // Threads move pairs of neighbouring vectors (32 bytes, never across a tile row)
    // with 256-bit accesses: kLinearUnroll / 2 pairs per thread, one 16 KiB chunk per CTA.
    constexpr uint32_t kTilePairs = kTileVectors / 2;             // 16 or 32
    constexpr uint32_t kPairsPerRow = kVectorsPerRow / 2;         // 1 or 2
    constexpr int kPairUnroll = kLinearUnroll / 2;
    constexpr uint64_t kChunk = static_cast<uint64_t>(kLinearThreads) * kPairUnroll;
    const uint64_t pairs = p.vectors / 2;                         // whole tiles: always even
    const uint64_t chunks = (pairs + kChunk - 1) / kChunk;
    for (uint64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
        const uint64_t base = chunk * kChunk + threadIdx.x;
        uint4 a[kPairUnroll][2], b[kPairUnroll][2];
#pragma unroll
        for (int u = 0; u < kPairUnroll; ++u) {
            const uint64_t index = base + u * kLinearThreads;
            if (index < pairs) {
                load_u8_stream(p.big + 2 * index, &a[u][0], &a[u][1]);
                const uint32_t tile = static_cast<uint32_t>(index / kTilePairs);
                const uint32_t in_tile = static_cast<uint32_t>(index % kTilePairs);
                if constexpr (!COLUMN) {
                    const uint32_t tc = p.cols_shift < 32 ? tile & ((1u << p.cols_shift) - 1u)
                                                          : tile % p.tile_cols;
                    const uint4* row0 = reinterpret_cast<const uint4*>(
                            p.small + static_cast<size_t>(tc) * kTileSlots * ELEM
                            + (in_tile % kPairsPerRow) * 32);
                    b[u][0] = __ldg(row0);
                    b[u][1] = __ldg(row0 + 1);
                } else {
                    uint32_t band = p.cols_shift < 32 ? tile >> p.cols_shift : tile / p.tile_cols;
                    if (!p.single_plane) band %= p.tile_rows;
                    const unsigned char* cell = p.small
                            + static_cast<size_t>(band) * kTileSlots * ELEM
                            + (in_tile / kPairsPerRow) * kTile * ELEM;
                    uint32_t value;
                    if constexpr (ELEM == 4) {
                        value = __ldg(reinterpret_cast<const uint32_t*>(cell));
                    } else {
                        const uint32_t half = __ldg(reinterpret_cast<const uint16_t*>(cell));
                        value = half | (half << 16);
                    }
                    b[u][0] = make_uint4(value, value, value, value);
                    b[u][1] = b[u][0];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kPairUnroll; ++u) {
            const uint64_t index = base + u * kLinearThreads;
            if (index < pairs) {
                store_u8_stream(p.out + 2 * index,
                                SMALL_IS_LHS ? apply_vector<L, OP>(b[u][0], a[u][0])
                                             : apply_vector<L, OP>(a[u][0], b[u][0]),
                                SMALL_IS_LHS ? apply_vector<L, OP>(b[u][1], a[u][1])
                                             : apply_vector<L, OP>(a[u][1], b[u][1]));
            }
        }
    }
}

template <Leaf L, int OP>
static int launch_stream_bc(const StreamBcParams& params, bool column, bool small_is_lhs,
                            cudaStream_t stream) {
    const uint64_t per_cta = static_cast<uint64_t>(kLinearThreads) * kLinearUnroll;
    const unsigned grid = grid_one_shot((params.vectors + per_cta - 1) / per_cta);
    if (column) {
        if (small_is_lhs) binary_stream_bc_kernel<L, OP, true, true><<<grid, kLinearThreads, 0, stream>>>(params);
        else binary_stream_bc_kernel<L, OP, true, false><<<grid, kLinearThreads, 0, stream>>>(params);
    } else {
        if (small_is_lhs) binary_stream_bc_kernel<L, OP, false, true><<<grid, kLinearThreads, 0, stream>>>(params);
        else binary_stream_bc_kernel<L, OP, false, false><<<grid, kLinearThreads, 0, stream>>>(params);
    }
    return check_launch("binary launch");
}

template <Leaf L>
static int launch_stream_bc_op(int op, const StreamBcParams& params, bool column,
                               bool small_is_lhs, cudaStream_t stream) {
    switch (op) {
        case IOMB_ADD: return launch_stream_bc<L, IOMB_ADD>(params, column, small_is_lhs, stream);
        case IOMB_MUL: return launch_stream_bc<L, IOMB_MUL>(params, column, small_is_lhs, stream);
        case IOMB_SUB: return launch_stream_bc<L, IOMB_SUB>(params, column, small_is_lhs, stream);
        default:
            if constexpr (L == Leaf::I32) {
                return fail(IOMB_ERR_UNSUPPORTED, "binary: integer division is not admitted");
            } else {
                return launch_stream_bc<L, IOMB_DIV>(params, column, small_is_lhs, stream);
            }
    }
}

// ---- tiled general kernel --------------------------------------------------

struct BinaryParams {
    Operand lhs;
    Operand rhs;
    Operand out;
    Leading leading;
    uint32_t rows;        // result rows
    uint32_t cols;        // result columns
    uint32_t tile_rows;   // result tile rows
    uint32_t tile_cols;   // result tile columns
    uint32_t run_tiles;   // tiles one warp handles per work item
    uint32_t runs;        // work items per band
    uint64_t items;       // planes * tile_rows * runs
};

constexpr int kTiledThreads = 256;
constexpr int kTiledWarps = kTiledThreads / 32;

// Per-item cursor of one operand for one lane vector: the address of the
// vector in tile column 0 of the operand's band plus the byte step per tile
// column (zero for a column-broadcast operand). A broadcast operand reads its
// row 0 / column 0 instead of the lane's own row / column.
struct Cursor {
    const unsigned char* address;
    uint32_t step;
    uint32_t scalar;   // column broadcast: replicate one element
};

template <int ELEM>
__device__ __forceinline__ Cursor make_cursor(
        const Operand& operand, uint64_t plane, uint32_t tr, uint32_t slot) {
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    const uint32_t row = operand.bc_rows ? 0u : slot / kTile;
    const uint32_t col = operand.bc_cols ? 0u : slot % kTile;
    const uint32_t otr = operand.bc_rows ? 0u : tr;
    Cursor cursor;
    cursor.address = operand.base
            + (plane * operand.tile_rows + otr) * operand.tile_cols
                    * static_cast<uint64_t>(kTileBytes)
            + (row * kTile + col) * ELEM;
    cursor.step = operand.bc_cols ? 0u : kTileBytes;
    cursor.scalar = operand.bc_cols;
    return cursor;
}

template <int ELEM>
__device__ __forceinline__ uint4 load_cursor(const Cursor& cursor, uint32_t tc) {
    const unsigned char* address = cursor.address + static_cast<uint64_t>(tc) * cursor.step;
    if (!cursor.scalar) return load_u4(address);
    if constexpr (ELEM == 4) {
        const uint32_t value = *reinterpret_cast<const uint32_t*>(address);
        return make_uint4(value, value, value, value);
    } else {
        const uint32_t half = *reinterpret_cast<const uint16_t*>(address);
        const uint32_t value = half | (half << 16);
        return make_uint4(value, value, value, value);
    }
}

template <int ELEM>
__device__ __forceinline__ void store_masked(
        unsigned char* address, uint4 value, uint32_t valid) {
    constexpr uint32_t kPerVector = 16 / ELEM;
    if (valid >= kPerVector) {
        store_u4(address, value);
        return;
    }
    const uint32_t words[4] = {value.x, value.y, value.z, value.w};
    if constexpr (ELEM == 4) {
        for (uint32_t e = 0; e < valid; ++e) {
            reinterpret_cast<uint32_t*>(address)[e] = words[e];
        }
    } else {
        for (uint32_t e = 0; e < valid; ++e) {
            reinterpret_cast<uint16_t*>(address)[e] =
                    static_cast<uint16_t>(words[e / 2] >> ((e & 1u) * 16));
        }
    }
}

template <Leaf L, int OP>
__global__ void __launch_bounds__(kTiledThreads)
binary_tiled_kernel(const BinaryParams p) {
    constexpr int ELEM = L == Leaf::BF16 ? 2 : 4;
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kVectorsPerLane = kTileBytes / 512;   // 1 (16-bit) or 2 (32-bit)
    constexpr uint32_t kPerVector = 16 / ELEM;
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kTiledWarps + (threadIdx.x >> 5);
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kTiledWarps;
    for (uint64_t item = warp; item < p.items; item += warps) {
        const uint32_t run = static_cast<uint32_t>(item % p.runs);
        const uint64_t band = item / p.runs;
        const uint32_t tr = static_cast<uint32_t>(band % p.tile_rows);
        const uint64_t index = band / p.tile_rows;
        const uint64_t lhs_plane = operand_plane(p.lhs, p.leading, index);
        const uint64_t rhs_plane = operand_plane(p.rhs, p.leading, index);
        const uint64_t out_plane = operand_plane(p.out, p.leading, index);
        const uint32_t first = run * p.run_tiles;
        const uint32_t last = min(first + p.run_tiles, p.tile_cols);
        unsigned char* out_band = p.out.base
                + (out_plane * p.out.tile_rows + tr) * p.out.tile_cols
                        * static_cast<uint64_t>(kTileBytes);
        const uint32_t rows_left = p.rows - tr * kTile;   // >= 1
        Cursor lhs_cursor[kVectorsPerLane], rhs_cursor[kVectorsPerLane];
#pragma unroll
        for (uint32_t v = 0; v < kVectorsPerLane; ++v) {
            const uint32_t slot = (v * 512 + lane * 16) / ELEM;
            lhs_cursor[v] = make_cursor<ELEM>(p.lhs, lhs_plane, tr, slot);
            rhs_cursor[v] = make_cursor<ELEM>(p.rhs, rhs_plane, tr, slot);
        }
        // kBatch tiles per iteration: four 16-byte loads per operand and lane
        // are in flight before the first store.
        constexpr uint32_t kBatch = 4 / kVectorsPerLane;
        for (uint32_t tc0 = first; tc0 < last; tc0 += kBatch) {
            uint4 a[kBatch][kVectorsPerLane], b[kBatch][kVectorsPerLane];
#pragma unroll
            for (uint32_t k = 0; k < kBatch; ++k) {
                const uint32_t tc = tc0 + k;
                if (tc < last) {
#pragma unroll
                    for (uint32_t v = 0; v < kVectorsPerLane; ++v) {
                        a[k][v] = load_cursor<ELEM>(lhs_cursor[v], tc);
                        b[k][v] = load_cursor<ELEM>(rhs_cursor[v], tc);
                    }
                }
            }
#pragma unroll
            for (uint32_t k = 0; k < kBatch; ++k) {
                const uint32_t tc = tc0 + k;
                if (tc < last) {
                    const uint32_t cols_left = p.cols - tc * kTile;   // >= 1
#pragma unroll
                    for (uint32_t v = 0; v < kVectorsPerLane; ++v) {
                        const uint32_t slot = (v * 512 + lane * 16) / ELEM;
                        const uint32_t row = slot / kTile;
                        const uint32_t col = slot % kTile;
                        if (row >= rows_left || col >= cols_left) continue;
                        const uint32_t valid = min(kPerVector, cols_left - col);
                        store_masked<ELEM>(
                                out_band + static_cast<uint64_t>(tc) * kTileBytes + slot * ELEM,
                                apply_vector<L, OP>(a[k][v], b[k][v]), valid);
                    }
                }
            }
        }
    }
}

// ---- host dispatch --------------------------------------------------------

template <Leaf L, int OP>
static int launch(const BinaryParams& params, bool linear, uint64_t linear_vectors,
                  cudaStream_t stream) {
    if (linear) {
        const uint64_t per_cta = static_cast<uint64_t>(kLinearThreads) * kLinearUnroll;
        const unsigned grid = grid_one_shot((linear_vectors + per_cta - 1) / per_cta);
        binary_linear_kernel<L, OP><<<grid, kLinearThreads, 0, stream>>>(
                reinterpret_cast<const uint4*>(params.lhs.base),
                reinterpret_cast<const uint4*>(params.rhs.base),
                reinterpret_cast<uint4*>(params.out.base), linear_vectors);
    } else {
        const unsigned grid = grid_one_shot((params.items + kTiledWarps - 1) / kTiledWarps);
        binary_tiled_kernel<L, OP><<<grid, kTiledThreads, 0, stream>>>(params);
    }
    return check_launch("binary launch");
}

template <Leaf L>
static int launch_op(int op, const BinaryParams& params, bool linear,
                     uint64_t linear_vectors, cudaStream_t stream) {
    switch (op) {
        case IOMB_ADD: return launch<L, IOMB_ADD>(params, linear, linear_vectors, stream);
        case IOMB_MUL: return launch<L, IOMB_MUL>(params, linear, linear_vectors, stream);
        case IOMB_SUB: return launch<L, IOMB_SUB>(params, linear, linear_vectors, stream);
        default:
            if constexpr (L == Leaf::I32) {
                return fail(IOMB_ERR_UNSUPPORTED, "binary: integer division is not admitted");
            } else {
                return launch<L, IOMB_DIV>(params, linear, linear_vectors, stream);
            }
    }
}

// ---- every other byte-multiple leaf: one thread per logical element ------------
//
// I8/U8, I16/U16, I64/U64 (wrapping ADD/MUL/SUB), F16 (one IEEE binary32
// operation, one RNE narrowing to binary16, positive quiet NaN 0x7E00: equal to the
// reference codec because 24 >= 2 * 11 + 2) and the two 8-bit floating leaves
// F8_E4M3FN / F8_E5M2 (decoded exactly to binary32, one binary32 operation, one encode
// by the codec's rules, see F8Format). These leaves are off the serving
// path, so the kernel is the simple one: thread e owns logical element e of the
// result, reads its two inputs through the same tile map the fast kernels use and
// writes one element; broadcast operands read their row 0 / column 0.
enum class Wide : int { Int8 = 0, Int16 = 1, Int64 = 2, Half = 3, F8E4M3 = 4, F8E5M2 = 5, Double = 6 };

template <Wide W>
struct WideTraits {
    static constexpr int kBytes =
            (W == Wide::Int8 || W == Wide::F8E4M3 || W == Wide::F8E5M2) ? 1
            : (W == Wide::Int64 || W == Wide::Double) ? 8 : 2;
};

template <int BYTES>
__device__ __forceinline__ uint64_t load_element(const unsigned char* address) {
    if constexpr (BYTES == 1) return *address;
    if constexpr (BYTES == 2) return *reinterpret_cast<const uint16_t*>(address);
    return *reinterpret_cast<const uint64_t*>(address);
}

template <int BYTES>
__device__ __forceinline__ void store_element(unsigned char* address, uint64_t value) {
    if constexpr (BYTES == 1) *address = static_cast<unsigned char>(value);
    else if constexpr (BYTES == 2) *reinterpret_cast<uint16_t*>(address) = static_cast<uint16_t>(value);
    else *reinterpret_cast<uint64_t*>(address) = value;
}

// The 8-bit floating formats as the reference codec defines them
// (src/shared/scalar_binary_codec.hpp:30-108). E4M3FN: bias 7, finite only, yet every code
// with all exponent bits set decodes as NaN, so the largest finite value is 240 (0x77),
// which is also what an overflow or an infinite result encodes to; NaN is 0x7F. E5M2: bias
// 15, infinities 0x7C / 0xFC, NaN 0x7E. Results are NaN-positive, zeros keep their sign,
// subnormals are kept, rounding is to nearest even.
//
// RESERVED = false is the codec's rule for the formats with fewer than four exponent bits
// (F4_E2M1, F6_E2M3, F6_E3M2): every code is a finite value, and an infinite or NaN result
// encodes to the largest value (a NaN to the positive one).
template <int EBITS, int FBITS, int BIAS, bool INFS, bool RESERVED = true>
struct F8Format {
    static constexpr uint32_t kExpMask = (1u << EBITS) - 1;
    static constexpr uint32_t kFracMask = (1u << FBITS) - 1;
    static constexpr uint32_t kTopExp = kExpMask - (RESERVED ? 1u : 0u);   // largest finite exponent field
    static constexpr int kMinSub = 1 - BIAS - FBITS;            // exponent of the smallest subnormal
    static constexpr int kMaxExp = static_cast<int>(kTopExp) - BIAS;
    static constexpr uint32_t kOverflow = INFS ? kExpMask << FBITS : (kTopExp << FBITS) | kFracMask;
    static constexpr uint32_t kNan = !RESERVED ? kOverflow
            : (kExpMask << FBITS) | (INFS ? 1u << (FBITS - 1) : kFracMask);

    __device__ static float decode(uint32_t raw) {
        const uint32_t sign = (raw >> (EBITS + FBITS)) & 1u;
        const uint32_t exponent = (raw >> FBITS) & kExpMask;
        const uint32_t fraction = raw & kFracMask;
        float value;
        if (RESERVED && exponent == kExpMask) {
            value = (INFS && fraction == 0) ? __uint_as_float(0x7f800000u) : __uint_as_float(0x7fc00000u);
        } else if (exponent == 0) {
            value = __fmul_rn(__uint2float_rn(fraction),
                              __uint_as_float(static_cast<uint32_t>(kMinSub + 127) << 23));
        } else {
            value = __fmul_rn(__uint2float_rn((1u << FBITS) + fraction),
                              __uint_as_float((exponent + 127u - BIAS - FBITS) << 23));
        }
        return sign ? -value : value;
    }

    // `value` is a binary32 result of one operation on two decoded operands: zero, normal,
    // infinite or NaN (the smallest nonzero magnitude, 2^-32, is far above binary32's
    // subnormal range).
    __device__ static uint32_t encode(float value) {
        if (value != value) return kNan;
        const uint32_t bits = __float_as_uint(value);
        const uint32_t sign = (bits >> 31) << (EBITS + FBITS);
        const uint32_t magnitude = bits & 0x7fffffffu;
        if (magnitude == 0x7f800000u) return sign | kOverflow;
        if (magnitude == 0) return sign;
        int exponent = static_cast<int>(magnitude >> 23) - 127;
        const uint32_t significand = (magnitude & 0x007fffffu) | 0x00800000u;   // 24 bits
        if (exponent < kMinSub + FBITS) {
            // q = RNE(value * 2^-kMinSub); q == 2^FBITS is the smallest normal's code
            const int shift = 23 + kMinSub - exponent;
            if (shift > 25) return sign;
            const uint32_t kept = significand >> shift;
            const uint32_t rest = significand & ((1u << shift) - 1u);
            const uint32_t half = 1u << (shift - 1);
            return sign | (kept + ((rest > half || (rest == half && (kept & 1u))) ? 1u : 0u));
        }
        if (exponent > kMaxExp) return sign | kOverflow;
        constexpr int kShift = 23 - FBITS;
        uint32_t kept = significand >> kShift;                    // 1.fraction, FBITS + 1 bits
        const uint32_t rest = significand & ((1u << kShift) - 1u);
        constexpr uint32_t kHalf = 1u << (kShift - 1);
        kept += (rest > kHalf || (rest == kHalf && (kept & 1u))) ? 1u : 0u;
        if (kept == (2u << FBITS)) {
            kept = 1u << FBITS;
            ++exponent;
        }
        if (exponent > kMaxExp) return sign | kOverflow;
        return sign | (static_cast<uint32_t>(exponent + BIAS) << FBITS) | (kept & kFracMask);
    }
};
using F8E4M3Format = F8Format<4, 3, 7, false>;
using F8E5M2Format = F8Format<5, 2, 15, true>;
using F4E2M1Format = F8Format<2, 1, 1, false, false>;
using F6E2M3Format = F8Format<2, 3, 1, false, false>;
using F6E3M2Format = F8Format<3, 2, 3, false, false>;

template <Wide W, int OP>
__device__ __forceinline__ uint64_t apply_wide(uint64_t a, uint64_t b) {
    if constexpr (W == Wide::F8E4M3 || W == Wide::F8E5M2) {
        using Format = typename std::conditional<W == Wide::F8E4M3, F8E4M3Format, F8E5M2Format>::type;
        const float r = apply_f32<OP>(Format::decode(static_cast<uint32_t>(a)),
                                      Format::decode(static_cast<uint32_t>(b)));
        return Format::encode(r);
    } else if constexpr (W == Wide::Double) {
        // One IEEE binary64 operation, correctly rounded: the carrier of the reference's own
        // GPU kernels (src/shared/standard_tiled_add.inl:110-116). The reference CPU backend
        // computes in x87 extended precision and rounds a second time, which can differ in
        // the last place (64 < 2 * 53 + 2); the bound is one code, measured in the tests.
        const double x = __longlong_as_double(static_cast<long long>(a));
        const double y = __longlong_as_double(static_cast<long long>(b));
        const double r = OP == IOMB_ADD ? __dadd_rn(x, y) : OP == IOMB_MUL ? __dmul_rn(x, y)
                : OP == IOMB_SUB ? __dsub_rn(x, y) : __ddiv_rn(x, y);
        if (r != r) return 0x7FF8000000000000ull;
        return static_cast<uint64_t>(__double_as_longlong(r));
    } else if constexpr (W == Wide::Half) {
        const float x = __half2float(__ushort_as_half(static_cast<unsigned short>(a)));
        const float y = __half2float(__ushort_as_half(static_cast<unsigned short>(b)));
        const float r = apply_f32<OP>(x, y);
        if (r != r) return 0x7E00u;
        return __half_as_ushort(__float2half_rn(r));
    } else {
        // Wrapping: the low bits of the 64-bit result are the result of every narrower width.
        return OP == IOMB_ADD ? a + b : OP == IOMB_MUL ? a * b : a - b;
    }
}

template <Wide W, int OP>
__global__ void __launch_bounds__(kTiledThreads)
binary_element_kernel(const BinaryParams p, uint64_t elements) {
    constexpr int BYTES = WideTraits<W>::kBytes;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kTiledThreads;
    for (uint64_t e = static_cast<uint64_t>(blockIdx.x) * kTiledThreads + threadIdx.x; e < elements;
         e += stride) {
        const uint32_t col = static_cast<uint32_t>(e % p.cols);
        const uint64_t rest = e / p.cols;
        const uint32_t row = static_cast<uint32_t>(rest % p.rows);
        const uint64_t index = rest / p.rows;
        auto slot = [&](const Operand& operand) {
            const uint32_t r = operand.bc_rows ? 0u : row;
            const uint32_t c = operand.bc_cols ? 0u : col;
            const uint64_t plane = operand_plane(operand, p.leading, index);
            const uint64_t tile = (plane * operand.tile_rows + r / kTile) * operand.tile_cols + c / kTile;
            return operand.base + (tile * kTileSlots + (r % kTile) * kTile + c % kTile) * BYTES;
        };
        const uint64_t a = load_element<BYTES>(slot(p.lhs));
        const uint64_t b = load_element<BYTES>(slot(p.rhs));
        store_element<BYTES>(const_cast<unsigned char*>(slot(p.out)), apply_wide<W, OP>(a, b));
    }
}

// ---- leaves narrower than a byte: one thread per 16-element tile row -------------
//
// I2/U2, I4/U4 (wrapping) and F4_E2M1, F6_E2M3, F6_E3M2 (decode, one binary32 operation,
// encode). Slots are packed LSB first (src/tensor.cpp:136-164 gives the slot, the slot
// times the leaf width the bit), so a tile row of 16 slots is 4, 8 or 12 whole bytes on a
// 4-byte boundary: the thread that owns it reads it, replaces the logical columns and
// writes it back, and the bits of padding columns survive. Inputs are fetched element by
// element through the tile map (broadcast operands read their row 0 / column 0).
enum class Narrow : int { Int = 0, F4E2M1 = 1, F6E2M3 = 2, F6E3M2 = 3 };

template <int BITS, Narrow KIND, int OP>
__device__ __forceinline__ uint32_t apply_narrow(uint32_t a, uint32_t b) {
    if constexpr (KIND == Narrow::Int) {
        const uint32_t r = OP == IOMB_ADD ? a + b : OP == IOMB_MUL ? a * b : a - b;
        return r & ((1u << BITS) - 1u);
    } else {
        using Format = typename std::conditional<KIND == Narrow::F4E2M1, F4E2M1Format,
                typename std::conditional<KIND == Narrow::F6E2M3, F6E2M3Format, F6E3M2Format>::type>::type;
        return Format::encode(apply_f32<OP>(Format::decode(a), Format::decode(b)));
    }
}

template <int BITS>
__device__ __forceinline__ uint32_t fetch_narrow(const Operand& operand, const Leading& leading,
                                                 uint64_t index, uint32_t row, uint32_t col) {
    const uint32_t r = operand.bc_rows ? 0u : row;
    const uint32_t c = operand.bc_cols ? 0u : col;
    const uint64_t plane = operand_plane(operand, leading, index);
    const uint64_t tile = (plane * operand.tile_rows + r / kTile) * operand.tile_cols + c / kTile;
    const uint64_t bit = (tile * kTileSlots + (r % kTile) * kTile + c % kTile) * BITS;
    const unsigned char* byte = operand.base + (bit >> 3);
    const uint32_t shift = static_cast<uint32_t>(bit & 7u);
    uint32_t value = static_cast<uint32_t>(byte[0]) >> shift;
    if (shift + BITS > 8) value |= static_cast<uint32_t>(byte[1]) << (8 - shift);
    return value & ((1u << BITS) - 1u);
}

template <int BITS, Narrow KIND, int OP>
__global__ void __launch_bounds__(kTiledThreads)
binary_narrow_kernel(const BinaryParams p, uint64_t items) {
    constexpr int kWords = BITS / 2;                 // 32-bit words of one tile row
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kTiledThreads;
    for (uint64_t item = static_cast<uint64_t>(blockIdx.x) * kTiledThreads + threadIdx.x; item < items;
         item += stride) {
        const uint32_t tc = static_cast<uint32_t>(item % p.tile_cols);
        const uint64_t rest = item / p.tile_cols;
        const uint32_t row = static_cast<uint32_t>(rest % p.rows);
        const uint64_t index = rest / p.rows;
        const uint32_t live = min(kTile, p.cols - tc * kTile);
        const uint64_t out_tile = (operand_plane(p.out, p.leading, index) * p.out.tile_rows + row / kTile)
                * p.out.tile_cols + tc;
        uint32_t* words = reinterpret_cast<uint32_t*>(
                p.out.base + (out_tile * kTileSlots + (row % kTile) * kTile) * BITS / 8);
        unsigned __int128 packed = 0;
#pragma unroll
        for (int w = 0; w < kWords; ++w) packed |= static_cast<unsigned __int128>(words[w]) << (32 * w);
        for (uint32_t c = 0; c < live; ++c) {
            const uint32_t col = tc * kTile + c;
            const uint32_t a = fetch_narrow<BITS>(p.lhs, p.leading, index, row, col);
            const uint32_t b = fetch_narrow<BITS>(p.rhs, p.leading, index, row, col);
            const unsigned __int128 mask = static_cast<unsigned __int128>((1u << BITS) - 1u) << (c * BITS);
            packed = (packed & ~mask)
                    | (static_cast<unsigned __int128>(apply_narrow<BITS, KIND, OP>(a, b)) << (c * BITS));
        }
#pragma unroll
        for (int w = 0; w < kWords; ++w) words[w] = static_cast<uint32_t>(packed >> (32 * w));
    }
}

template <int BITS, Narrow KIND>
static int launch_narrow(int op, const BinaryParams& params, cudaStream_t stream) {
    const uint64_t items = params.leading.planes * params.rows * params.tile_cols;
    const unsigned grid = grid_for((items + kTiledThreads - 1) / kTiledThreads, 16);
    switch (op) {
        case IOMB_ADD: binary_narrow_kernel<BITS, KIND, IOMB_ADD><<<grid, kTiledThreads, 0, stream>>>(params, items); break;
        case IOMB_MUL: binary_narrow_kernel<BITS, KIND, IOMB_MUL><<<grid, kTiledThreads, 0, stream>>>(params, items); break;
        case IOMB_SUB: binary_narrow_kernel<BITS, KIND, IOMB_SUB><<<grid, kTiledThreads, 0, stream>>>(params, items); break;
        default:
            if constexpr (KIND != Narrow::Int) {
                binary_narrow_kernel<BITS, KIND, IOMB_DIV><<<grid, kTiledThreads, 0, stream>>>(params, items);
            } else {
                return fail(IOMB_ERR_UNSUPPORTED, "binary: integer division is not admitted");
            }
    }
    return check_launch("binary launch");
}

template <Wide W>
static int launch_element(int op, const BinaryParams& params, cudaStream_t stream) {
    const uint64_t elements = params.leading.planes * params.rows * params.cols;
    const unsigned grid = grid_for((elements + kTiledThreads - 1) / kTiledThreads, 16);
    switch (op) {
        case IOMB_ADD: binary_element_kernel<W, IOMB_ADD><<<grid, kTiledThreads, 0, stream>>>(params, elements); break;
        case IOMB_MUL: binary_element_kernel<W, IOMB_MUL><<<grid, kTiledThreads, 0, stream>>>(params, elements); break;
        case IOMB_SUB: binary_element_kernel<W, IOMB_SUB><<<grid, kTiledThreads, 0, stream>>>(params, elements); break;
        default:
            if constexpr (W == Wide::Half || W == Wide::F8E4M3 || W == Wide::F8E5M2
                          || W == Wide::Double) {
                binary_element_kernel<W, IOMB_DIV><<<grid, kTiledThreads, 0, stream>>>(params, elements);
            } else {
                return fail(IOMB_ERR_UNSUPPORTED, "binary: integer division is not admitted");
            }
    }
    return check_launch("binary launch");
}

}  // namespace iomb

extern "C" int iomb_binary_supported(uint32_t dtype) {
    return dtype != IOMB_BOOL && dtype != IOMB_F8_E8M0 && iomb_dtype_bits(dtype) != 0 ? 1 : 0;
}

extern "C" int iomb_binary(int op, const iomb_view* lhs, const iomb_view* rhs,
                           const iomb_view* out, void* stream) {
    using namespace iomb;
    if (op < IOMB_ADD || op > IOMB_DIV) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "binary: unknown operation");
    }
    ViewFacts fl{}, fr{}, fo{};
    int status = check_view(lhs, "binary lhs", &fl);
    if (status == IOMB_OK) status = check_view(rhs, "binary rhs", &fr);
    if (status == IOMB_OK) status = check_view(out, "binary out", &fo);
    if (status != IOMB_OK) return status;
    if (lhs->dtype != rhs->dtype || lhs->dtype != out->dtype) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "binary specifications do not match");
    }
    // Right-aligned broadcast shape (src/device_ops_binary.cpp:121-143).
    const uint32_t rank = lhs->rank > rhs->rank ? lhs->rank : rhs->rank;
    uint64_t result[IOMB_MAX_RANK];
    for (uint32_t i = 0; i < rank; ++i) {
        const uint64_t la = i < rank - lhs->rank ? 1 : lhs->dims[i - (rank - lhs->rank)];
        const uint64_t ra = i < rank - rhs->rank ? 1 : rhs->dims[i - (rank - rhs->rank)];
        if (la != ra && la != 1 && ra != 1) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "binary shapes are not broadcast compatible");
        }
        result[i] = la > ra ? la : ra;
    }
    if (out->rank != rank) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "binary output shape is incorrect");
    }
    for (uint32_t i = 0; i < rank; ++i) {
        if (out->dims[i] != result[i]) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "binary output shape is incorrect");
        }
    }
    // Aligned plane strides, zero on broadcast axes (snapshot_binary_view,
    // src/device_ops_binary.cpp:61-100).
    const uint32_t lead_rank = rank - 2;
    const iomb_view* views[3] = {lhs, rhs, out};
    uint64_t strides[3][kMaxLead] = {};
    bool broadcasts[3] = {false, false, false};
    for (int k = 0; k < 3; ++k) {
        const uint32_t offset = rank - views[k]->rank;
        broadcasts[k] = offset != 0;
        for (uint32_t axis = 0; axis < lead_rank; ++axis) {
            if (axis < offset) {
                broadcasts[k] = broadcasts[k] || result[axis] != 1;
                continue;
            }
            const uint32_t source_axis = axis - offset;
            if (views[k]->dims[source_axis] == 1 && result[axis] != 1) {
                broadcasts[k] = true;
                continue;
            }
            strides[k][axis] = views[k]->plane_strides[source_axis];
        }
    }
    const bool lhs_bc_rows = fl.rows == 1 && result[rank - 2] != 1;
    const bool rhs_bc_rows = fr.rows == 1 && result[rank - 2] != 1;
    const bool lhs_bc_cols = fl.cols == 1 && result[rank - 1] != 1;
    const bool rhs_bc_cols = fr.cols == 1 && result[rank - 1] != 1;
    broadcasts[0] = broadcasts[0] || lhs_bc_rows || lhs_bc_cols;
    broadcasts[1] = broadcasts[1] || rhs_bc_rows || rhs_bc_cols;
    // Alias rule (src/device_ops_binary.cpp:152-169): an input that shares the
    // output's owner must be exactly the output window and must not broadcast.
    const iomb_view* inputs[2] = {lhs, rhs};
    for (int k = 0; k < 2; ++k) {
        if (inputs[k]->base == out->base
                && (broadcasts[k] || !same_window(*inputs[k], *out))) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "binary input/output alias is forbidden");
        }
    }
    Leaf leaf = Leaf::I32;
    int wide = -1;      // a Wide ordinal when the leaf takes the per-element kernel
    int narrow = -1;    // 0..4 when the leaf is narrower than a byte
    switch (out->dtype) {
        case IOMB_I2: case IOMB_U2: narrow = 0; break;
        case IOMB_I4: case IOMB_U4: narrow = 1; break;
        case IOMB_F4_E2M1: narrow = 2; break;
        case IOMB_F6_E2M3: narrow = 3; break;
        case IOMB_F6_E3M2: narrow = 4; break;
        case IOMB_I32: case IOMB_U32: leaf = Leaf::I32; break;
        case IOMB_F32: leaf = Leaf::F32; break;
        case IOMB_BF16: leaf = Leaf::BF16; break;
        case IOMB_I8: case IOMB_U8: wide = static_cast<int>(Wide::Int8); break;
        case IOMB_I16: case IOMB_U16: wide = static_cast<int>(Wide::Int16); break;
        case IOMB_I64: case IOMB_U64: wide = static_cast<int>(Wide::Int64); break;
        case IOMB_F16: wide = static_cast<int>(Wide::Half); break;
        case IOMB_F8_E4M3FN: wide = static_cast<int>(Wide::F8E4M3); break;
        case IOMB_F8_E5M2: wide = static_cast<int>(Wide::F8E5M2); break;
        case IOMB_F64: wide = static_cast<int>(Wide::Double); break;
        default:
            return fail(IOMB_ERR_UNSUPPORTED, "binary: leaf is BOOL or F8_E8M0");
    }

    BinaryParams params{};
    collapse_leading(lead_rank, result, strides, 3, &params.leading);
    params.lhs = make_operand(*lhs, fl, strides[0], params.leading, lhs_bc_rows, lhs_bc_cols);
    params.rhs = make_operand(*rhs, fr, strides[1], params.leading, rhs_bc_rows, rhs_bc_cols);
    params.out = make_operand(*out, fo, strides[2], params.leading, false, false);
    params.rows = static_cast<uint32_t>(fo.rows);
    params.cols = static_cast<uint32_t>(fo.cols);
    if (fo.rows > 0xFFFFFFFFull || fo.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "binary: matrix extent exceeds the kernel limit");
    }
    params.tile_rows = static_cast<uint32_t>(fo.tile_rows);
    params.tile_cols = static_cast<uint32_t>(fo.tile_cols);
    params.run_tiles = fo.bytes == 2 ? 16u : 8u;   // 8 KiB of output per work item
    params.runs = (params.tile_cols + params.run_tiles - 1) / params.run_tiles;
    params.items = params.leading.planes * params.tile_rows * params.runs;

    if (narrow >= 0) {
        cudaStream_t narrow_stream = static_cast<cudaStream_t>(stream);
        switch (narrow) {
            case 0: return launch_narrow<2, Narrow::Int>(op, params, narrow_stream);
            case 1: return launch_narrow<4, Narrow::Int>(op, params, narrow_stream);
            case 2: return launch_narrow<4, Narrow::F4E2M1>(op, params, narrow_stream);
            case 3: return launch_narrow<6, Narrow::F6E2M3>(op, params, narrow_stream);
            default: return launch_narrow<6, Narrow::F6E3M2>(op, params, narrow_stream);
        }
    }
    if (wide >= 0) {
        cudaStream_t element_stream = static_cast<cudaStream_t>(stream);
        switch (static_cast<Wide>(wide)) {
            case Wide::Int8: return launch_element<Wide::Int8>(op, params, element_stream);
            case Wide::Int16: return launch_element<Wide::Int16>(op, params, element_stream);
            case Wide::Int64: return launch_element<Wide::Int64>(op, params, element_stream);
            case Wide::F8E4M3: return launch_element<Wide::F8E4M3>(op, params, element_stream);
            case Wide::F8E5M2: return launch_element<Wide::F8E5M2>(op, params, element_stream);
            case Wide::Double: return launch_element<Wide::Double>(op, params, element_stream);
            default: return launch_element<Wide::Half>(op, params, element_stream);
        }
    }
    const bool full = !broadcasts[0] && !broadcasts[1];
    const bool tile_multiple = fo.rows % kTile == 0 && fo.cols % kTile == 0;
    const bool linear = full && tile_multiple && params.leading.contiguous;
    uint64_t linear_vectors = 0;
    if (linear) {
        // Dense planes: advance each base to its first plane and stream.
        params.lhs.base += lhs->plane_offset * fl.plane_bytes;
        params.rhs.base += rhs->plane_offset * fr.plane_bytes;
        params.out.base += out->plane_offset * fo.plane_bytes;
        linear_vectors = params.leading.planes * fo.plane_bytes / 16;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // One dense full-shape operand against a single broadcast row or column plane.
    if (!linear && tile_multiple && broadcasts[0] != broadcasts[1]
            && fo.tile_rows * fo.tile_cols * params.leading.planes < 0xFFFFFFFFull) {
        const int small_index = broadcasts[0] ? 0 : 1;
        const int big_index = 1 - small_index;
        const iomb_view* small_view = small_index == 0 ? lhs : rhs;
        const iomb_view* big_view = big_index == 0 ? lhs : rhs;
        const ViewFacts& fs = small_index == 0 ? fl : fr;
        const ViewFacts& fb = big_index == 0 ? fl : fr;
        const bool row_form = fs.rows == 1 && fs.cols == fo.cols && fo.rows != 1;
        const bool col_form = fs.cols == 1 && fs.rows == fo.rows && fo.cols != 1;
        bool small_single = true;       // every leading axis of the small operand broadcasts
        bool dense = true;              // big and out advance one plane per logical plane
        const Operand& small_operand = small_index == 0 ? params.lhs : params.rhs;
        const Operand& big_operand = big_index == 0 ? params.lhs : params.rhs;
        for (uint32_t axis = 0; axis < params.leading.count; ++axis) {
            if (small_operand.stride[axis] != 0) small_single = false;
        }
        if (params.leading.count > 1) dense = false;
        if (params.leading.count == 1
                && (big_operand.stride[0] != 1 || params.out.stride[0] != 1)) {
            dense = false;
        }
        if ((row_form || col_form) && small_single && dense) {
            StreamBcParams stream_params{};
            stream_params.big = reinterpret_cast<const uint4*>(
                    static_cast<unsigned char*>(big_view->base) + big_view->plane_offset * fb.plane_bytes);
            stream_params.small = static_cast<const unsigned char*>(small_view->base)
                    + small_view->plane_offset * fs.plane_bytes;
            stream_params.out = reinterpret_cast<uint4*>(
                    static_cast<unsigned char*>(out->base) + out->plane_offset * fo.plane_bytes);
            stream_params.vectors = params.leading.planes * fo.plane_bytes / 16;
            stream_params.tile_rows = static_cast<uint32_t>(fo.tile_rows);
            stream_params.tile_cols = static_cast<uint32_t>(fo.tile_cols);
            stream_params.cols_shift = 32;
            if ((fo.tile_cols & (fo.tile_cols - 1)) == 0) {
                uint32_t shift = 0;
                while ((1ull << shift) < fo.tile_cols) ++shift;
                stream_params.cols_shift = shift;
            }
            stream_params.single_plane = params.leading.planes == 1 ? 1u : 0u;
            switch (leaf) {
                case Leaf::I32:
                    return launch_stream_bc_op<Leaf::I32>(op, stream_params, col_form, small_index == 0, s);
                case Leaf::F32:
                    return launch_stream_bc_op<Leaf::F32>(op, stream_params, col_form, small_index == 0, s);
                default:
                    return launch_stream_bc_op<Leaf::BF16>(op, stream_params, col_form, small_index == 0, s);
            }
        }
    }
    switch (leaf) {
        case Leaf::I32: return launch_op<Leaf::I32>(op, params, linear, linear_vectors, s);
        case Leaf::F32: return launch_op<Leaf::F32>(op, params, linear, linear_vectors, s);
        default: return launch_op<Leaf::BF16>(op, params, linear, linear_vectors, s);
    }
}
