// RMS normalization (optionally fused with the preceding residual ADD) on
// tiled storage.
//
// Replaces standard_tiled_rmsnorm_kernel (src/shared/standard_tiled_rmsnorm.inl:437-637),
// which runs one block per logical row over 32-byte pieces at a one-tile stride
// and re-reads x from global memory for its second pass. Here the unit of work
// is a group of g rows of one 16-row band (g = 16 when the band fits the
// staging buffer): its tiles are contiguous in memory, so the whole unit is
// brought into shared memory once with full-width coalesced copies, reduced
// there, normalised from there and written back with 16-byte stores. x is read
// from HBM exactly once.
//
// Arithmetic (src/cpu/queue.cpp:1145-1244): FP32 sum of individually rounded
// squares over the logical features only, mean = sum / F, + eps, true sqrt and
// true division, (x * inv) * w with both products rounded, NaN sign cleared, one
// RNE encode. Two accumulation orders are offered:
//   LANES16     16 column accumulators per row filled in tile order, combined
//               by the tree of src/cpu/avx512_bf16_rmsnorm_reduction.cpp:69-81
//               (the order of the reference's AVX-512 BF16 build);
//   SEQUENTIAL  one accumulator per row in feature order (the portable build).
// Rows holding an infinity or a NaN give the same result in either order, so
// the reference's per-row fallback (reduction.cpp:109-129) needs no branch.
#include "rmsnorm.cuh"

#include <stdio.h>
#include <stdlib.h>

namespace iomb {

constexpr int kRmsThreads = 256;
constexpr uint32_t kUnitCapBytes = 64 * 1024;

// Shared memory of one CTA:
//   [unit : tile_cols * G * 16 * ELEM bytes]  the staged rows of x, tile by tile
//   [unit2: same size, fused only]            the staged rows of the residual
//   [scale: tile_cols * 16 floats, SCALE_SMEM only] row 0 of the scale tiles, widened
//   [lanes: 16 x 16 floats][inverse: 16 floats][clean: 16 x uint32]
//
// G (rows per unit) is a template parameter so that every index split below is a
// shift. Thread t always owns the same (row, column group) of every tile it
// touches: vector v = t % (G * ELEM) of tiles t / (G * ELEM) + k * 256 / (G * ELEM).
// Every global read of x (and the residual) is an asynchronous 16-byte copy
// into shared memory, so a CTA has its whole unit in flight at once.
template <int ELEM, int G, bool FUSED, bool SCALE_SMEM>
__global__ void __launch_bounds__(kRmsThreads)
rmsnorm_kernel(const RmsParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kRowBytes = kTile * ELEM;             // one in-tile row
    constexpr uint32_t kVectorsPerRow = kRowBytes / 16;      // 2 (16-bit) or 4 (32-bit)
    constexpr uint32_t kPerVector = 16 / ELEM;
    constexpr uint32_t kPieceBytes = G * kRowBytes;          // per tile
    constexpr uint32_t kPieceVectors = G * kVectorsPerRow;   // 2 .. 64, divides 256
    constexpr uint32_t kTilesPerStep = kRmsThreads / kPieceVectors;
    const size_t unit_bytes = static_cast<size_t>(p.tile_cols) * kPieceBytes;
    const size_t buffer_bytes = (FUSED ? 2 : 1) * unit_bytes;
    float* scale = reinterpret_cast<float*>(smem + buffer_bytes);
    float* lanes = scale + (SCALE_SMEM ? static_cast<size_t>(p.tile_cols) * kTile : 0);
    float* inverse = lanes + kTile * kTile;
    uint32_t* clean = reinterpret_cast<uint32_t*>(inverse + kTile);
    const uint32_t tid = threadIdx.x;
    const uint32_t v = tid % kPieceVectors;                  // vector inside a piece
    const uint32_t tile0 = tid / kPieceVectors;
    const uint32_t row = v / kVectorsPerRow;                 // row inside the unit
    const uint32_t cv = v % kVectorsPerRow;
    const uint32_t col_in_tile = cv * kPerVector;
    const uint32_t full_tiles = p.cols / kTile;
    const uint32_t tail_cols = p.cols % kTile;
    __shared__ uint32_t scale_not_finite;

    // Where unit u lives: band (tile row, logical plane) and first in-tile row.
    struct Unit {
        uint32_t tr;
        uint32_t row0;
        uint32_t rows_in_band;
        uint64_t index;
        bool valid;
    };
    // 16 / G groups per band is a power of two; the band arithmetic is 32-bit
    // whenever the band count allows (64-bit division costs a hundred instructions
    // on every CTA's critical path).
    constexpr uint32_t kGroupsPerBand = kTile / G;
    auto locate = [&](uint64_t u) {
        Unit unit_at;
        const uint32_t group = static_cast<uint32_t>(u % kGroupsPerBand);
        const uint64_t band = u / kGroupsPerBand;
        if (band <= 0xFFFFFFFFull) {
            const uint32_t band32 = static_cast<uint32_t>(band);
            unit_at.tr = band32 % p.tile_rows;
            unit_at.index = band32 / p.tile_rows;
        } else {
            unit_at.tr = static_cast<uint32_t>(band % p.tile_rows);
            unit_at.index = band / p.tile_rows;
        }
        unit_at.row0 = group * G;
        unit_at.rows_in_band = min(kTile, p.rows - unit_at.tr * kTile);
        unit_at.valid = unit_at.row0 < unit_at.rows_in_band;     // uniform per CTA
        return unit_at;
    };
    // Address of this thread's vector in tile column 0 of the unit, per operand.
    auto band_base = [&](const Operand& operand, const Unit& at) {
        const uint64_t plane = operand_plane(operand, p.leading, at.index);
        return operand.base
                + (plane * operand.tile_rows + at.tr) * operand.tile_cols
                        * static_cast<uint64_t>(kTileBytes)
                + static_cast<size_t>(at.row0) * kRowBytes + v * 16;
    };
    // Starts the asynchronous copies of one unit into one staging buffer.
    auto issue = [&](uint64_t u, unsigned char* buffer) {
        const Unit at = locate(u);
        if (!at.valid) return;
        const unsigned char* x_cursor = band_base(p.x, at);
        for (uint32_t tile = tile0; tile < p.tile_cols; tile += kTilesPerStep) {
            cp_async_16(buffer + static_cast<size_t>(tile) * kPieceBytes + v * 16,
                        x_cursor + static_cast<size_t>(tile) * kTileBytes);
        }
        if constexpr (FUSED) {
            const unsigned char* r_cursor = band_base(p.residual, at);
            for (uint32_t tile = tile0; tile < p.tile_cols; tile += kTilesPerStep) {
                cp_async_16(buffer + unit_bytes + static_cast<size_t>(tile) * kPieceBytes + v * 16,
                            r_cursor + static_cast<size_t>(tile) * kTileBytes);
            }
        }
    };

    // The first unit's copies are issued before anything else so that they fly
    // while the scale row is staged.
    if (blockIdx.x < p.units) issue(blockIdx.x, smem);
    // Once per CTA: widen row 0 of every scale tile into shared memory (when it
    // fits) and note whether every logical scale value is finite.
    if (tid == 0) scale_not_finite = 0;
    __syncthreads();
    // One 16-byte vector of row 0 of a scale tile per step (2 or 4 vectors per tile).
    for (uint32_t k = tid; k < p.tile_cols * kVectorsPerRow; k += kRmsThreads) {
        const uint32_t tile = k / kVectorsPerRow, part = k % kVectorsPerRow;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
                p.scale_row + static_cast<size_t>(tile) * kTileBytes + part * 16));
        float w[kPerVector];
        if constexpr (ELEM == 2) {
            w[0] = bf16_lo(raw.x); w[1] = bf16_hi(raw.x); w[2] = bf16_lo(raw.y); w[3] = bf16_hi(raw.y);
            w[4] = bf16_lo(raw.z); w[5] = bf16_hi(raw.z); w[6] = bf16_lo(raw.w); w[7] = bf16_hi(raw.w);
        } else {
            w[0] = __uint_as_float(raw.x); w[1] = __uint_as_float(raw.y);
            w[2] = __uint_as_float(raw.z); w[3] = __uint_as_float(raw.w);
        }
        const uint32_t first = tile * kTile + part * kPerVector;
        bool finite = true;
#pragma unroll
        for (uint32_t e = 0; e < kPerVector; ++e) {
            // Padding columns of the last tile are not part of the scale.
            if (first + e < p.cols && !(fabsf(w[e]) <= 3.402823466e+38f)) finite = false;
        }
        if constexpr (SCALE_SMEM) {
            float4* target = reinterpret_cast<float4*>(scale + first);
            target[0] = make_float4(w[0], w[1], w[2], w[3]);
            if constexpr (ELEM == 2) target[1] = make_float4(w[4], w[5], w[6], w[7]);
        }
        if (!finite) scale_not_finite = 1;
    }
    __syncthreads();
    const bool scale_finite = scale_not_finite == 0;

    for (uint64_t u = blockIdx.x; u < p.units; u += gridDim.x) {
        unsigned char* unit = smem;
        unsigned char* unit2 = unit + unit_bytes;
        // ---- stage: every copy of the unit is in flight at once -------------
        if (u != blockIdx.x) issue(u, unit);
        cp_async_wait_all();
        const Unit at = locate(u);
        if (!at.valid) continue;
        const uint32_t live_rows = min(static_cast<uint32_t>(G), at.rows_in_band - at.row0);
        const bool row_live = row < live_rows;
        unsigned char* out_cursor = band_base(p.out, at);
        if constexpr (FUSED) {
            // Each thread adds the vectors it copied itself: sum = x + residual,
            // rounded to the leaf, kept in shared memory and stored.
            unsigned char* s_cursor = band_base(p.sum, at);
            for (uint32_t tile = tile0; tile < p.tile_cols; tile += kTilesPerStep) {
                unsigned char* slot = unit + static_cast<size_t>(tile) * kPieceBytes + v * 16;
                const uint4 total = add_vectors<ELEM>(
                        *reinterpret_cast<const uint4*>(slot),
                        *reinterpret_cast<const uint4*>(
                                unit2 + static_cast<size_t>(tile) * kPieceBytes + v * 16));
                *reinterpret_cast<uint4*>(slot) = total;
                const uint32_t col = tile * kTile + col_in_tile;
                if (row_live && col < p.cols) {
                    store_vector_masked<ELEM>(
                            s_cursor + static_cast<size_t>(tile) * kTileBytes, total,
                            min(kPerVector, p.cols - col));
                }
            }
        }
        __syncthreads();

        // ---- pass 1: row sums of squares ---------------------------------
        if (p.order == IOMB_RMS_LANES16) {
            if (tid < G * kTile) {
                const uint32_t chain_row = tid / kTile, lane = tid % kTile;
                const unsigned char* cursor = unit + (chain_row * kTile + lane) * ELEM;
                float acc = 0.0f;
#pragma unroll 8
                for (uint32_t tile = 0; tile < full_tiles; ++tile) {
                    acc = accumulate_square(acc, decode_element<ELEM>(cursor));
                    cursor += kPieceBytes;
                }
                if (lane < tail_cols) {
                    acc = accumulate_square(acc, decode_element<ELEM>(cursor));
                }
                lanes[chain_row * kTile + lane] = acc;
            }
            __syncthreads();
        }
        if (tid < G) {
            float sum;
            if (p.order == IOMB_RMS_LANES16) {
                sum = combine_lanes(lanes + tid * kTile);
            } else {
                const unsigned char* cursor = unit + tid * kRowBytes;
                sum = 0.0f;
                for (uint32_t tile = 0; tile < full_tiles; ++tile) {
#pragma unroll
                    for (uint32_t c = 0; c < kTile; ++c) {
                        sum = accumulate_square(sum, decode_element<ELEM>(cursor + c * ELEM));
                    }
                    cursor += kPieceBytes;
                }
                for (uint32_t c = 0; c < tail_cols; ++c) {
                    sum = accumulate_square(sum, decode_element<ELEM>(cursor + c * ELEM));
                }
            }
            inverse[tid] = row_inverse(sum, p.cols, p.eps);
            clean[tid] = row_is_clean(sum, scale_finite) ? 1u : 0u;
        }
        __syncthreads();

        // ---- pass 2: normalise, scale, encode, store ----------------------
        if (row_live) {
            const float inv = inverse[row];
            const bool fast = clean[row] != 0;
            auto emit = [&](uint32_t tile, uint32_t valid) {
                const uint4 xv = *reinterpret_cast<const uint4*>(
                        unit + static_cast<size_t>(tile) * kPieceBytes + v * 16);
                float w[kPerVector];
                if constexpr (SCALE_SMEM) {
                    const float* ws = scale + tile * kTile + col_in_tile;
                    const float4 w0 = *reinterpret_cast<const float4*>(ws);
                    w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
                    if constexpr (ELEM == 2) {
                        const float4 w1 = *reinterpret_cast<const float4*>(ws + 4);
                        w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
                    }
                } else {
                    // Large F: the scale row stays in global memory (L1-resident).
                    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
                            p.scale_row + static_cast<size_t>(tile) * kTileBytes + cv * 16));
                    if constexpr (ELEM == 2) {
                        w[0] = bf16_lo(raw.x); w[1] = bf16_hi(raw.x);
                        w[2] = bf16_lo(raw.y); w[3] = bf16_hi(raw.y);
                        w[4] = bf16_lo(raw.z); w[5] = bf16_hi(raw.z);
                        w[6] = bf16_lo(raw.w); w[7] = bf16_hi(raw.w);
                    } else {
                        w[0] = __uint_as_float(raw.x); w[1] = __uint_as_float(raw.y);
                        w[2] = __uint_as_float(raw.z); w[3] = __uint_as_float(raw.w);
                    }
                }
                const uint4 y = normalize_vector<ELEM>(xv, w, inv, fast);
                store_vector_masked<ELEM>(out_cursor + static_cast<size_t>(tile) * kTileBytes, y,
                                          valid);
            };
            uint32_t tile = tile0;
            for (; tile < full_tiles; tile += kTilesPerStep) emit(tile, kPerVector);
            if (tile == full_tiles && tail_cols > col_in_tile) {
                emit(tile, min(kPerVector, tail_cols - col_in_tile));
            }
        }
        __syncthreads();   // the unit buffer is reused by the next iteration
    }
    cp_async_wait_all();
}

// Rows too long for any staging (hundreds of KiB each): one CTA per row walks it twice
// in global memory. The 16 column accumulators (or the single one of the sequential
// order) are carried by sixteen threads (one) reading 2 or 4 bytes per tile, which is
// slow and only keeps every row length admissible, as the reference admits them all
// (src/device_ops_rmsnorm.cpp:75-127 has no feature limit).
template <int ELEM>
__global__ void __launch_bounds__(kRmsThreads)
rmsnorm_unstaged_kernel(const RmsParams p) {
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kRowBytes = kTile * ELEM;
    constexpr uint32_t kVectorsPerRow = kRowBytes / 16;
    constexpr uint32_t kPerVector = 16 / ELEM;
    __shared__ float lanes[kTile];
    __shared__ float inverse;
    const uint32_t tid = threadIdx.x;
    const uint32_t full_tiles = p.cols / kTile;
    const uint32_t tail_cols = p.cols % kTile;
    for (uint64_t u = blockIdx.x; u < p.units; u += gridDim.x) {
        const RmsUnit at = rms_locate<1>(p, u);
        if (!at.valid) continue;                              // uniform per CTA
        const unsigned char* row = rms_unit_base<ELEM>(p, p.x, at);
        unsigned char* out_row = rms_unit_base<ELEM>(p, p.out, at);
        if (p.order == IOMB_RMS_LANES16) {
            if (tid < kTile) {
                float acc = 0.0f;
                const unsigned char* cursor = row + tid * ELEM;
                for (uint32_t tile = 0; tile < full_tiles; ++tile) {
                    acc = accumulate_square(acc, decode_element<ELEM>(cursor));
                    cursor += kTileBytes;
                }
                if (tid < tail_cols) acc = accumulate_square(acc, decode_element<ELEM>(cursor));
                lanes[tid] = acc;
            }
            __syncthreads();
        }
        if (tid == 0) {
            float sum = 0.0f;
            if (p.order == IOMB_RMS_LANES16) {
                sum = combine_lanes(lanes);
            } else {
                const unsigned char* cursor = row;
                for (uint32_t tile = 0; tile <= full_tiles; ++tile) {
                    const uint32_t live = tile < full_tiles ? kTile : tail_cols;
                    for (uint32_t c = 0; c < live; ++c) {
                        sum = accumulate_square(sum, decode_element<ELEM>(cursor + c * ELEM));
                    }
                    cursor += kTileBytes;
                }
            }
            inverse = row_inverse(sum, p.cols, p.eps);
        }
        __syncthreads();
        const float inv = inverse;
        // One 16-byte vector per thread and step; the canonical-NaN path always.
        const uint32_t vectors = p.tile_cols * kVectorsPerRow;
        for (uint32_t k = tid; k < vectors; k += kRmsThreads) {
            const uint32_t tile = k / kVectorsPerRow, cv = k % kVectorsPerRow;
            const uint32_t col = tile * kTile + cv * kPerVector;
            if (col >= p.cols) continue;
            const uint4 xv = *reinterpret_cast<const uint4*>(
                    row + static_cast<size_t>(tile) * kTileBytes + cv * 16);
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
                    p.scale_row + static_cast<size_t>(tile) * kTileBytes + cv * 16));
            float w[kPerVector];
            widen_vector<ELEM>(raw, w);
            store_vector_masked<ELEM>(out_row + static_cast<size_t>(tile) * kTileBytes + cv * 16,
                                      normalize_vector<ELEM>(xv, w, inv, false),
                                      min(kPerVector, p.cols - col));
        }
        __syncthreads();
    }
}

using RmsKernel = void (*)(const RmsParams);

template <int ELEM, bool FUSED, bool SCALE_SMEM>
static RmsKernel pick_kernel(uint32_t g) {
    switch (g) {
        case 16: return rmsnorm_kernel<ELEM, 16, FUSED, SCALE_SMEM>;
        case 8: return rmsnorm_kernel<ELEM, 8, FUSED, SCALE_SMEM>;
        case 4: return rmsnorm_kernel<ELEM, 4, FUSED, SCALE_SMEM>;
        case 2: return rmsnorm_kernel<ELEM, 2, FUSED, SCALE_SMEM>;
        default: return rmsnorm_kernel<ELEM, 1, FUSED, SCALE_SMEM>;
    }
}

template <int ELEM>
static RmsKernel pick_kernel(uint32_t g, bool fused, bool scale_smem) {
    if (fused) {
        return scale_smem ? pick_kernel<ELEM, true, true>(g) : pick_kernel<ELEM, true, false>(g);
    }
    return scale_smem ? pick_kernel<ELEM, false, true>(g) : pick_kernel<ELEM, false, false>(g);
}


template <int ELEM, bool FUSED, bool SCALE_SMEM>
static int prepare_family() {
    for (uint32_t g = 1; g <= kTile; g *= 2) {
        const int status = allow_full_shared_memory(
                reinterpret_cast<const void*>(pick_kernel<ELEM, FUSED, SCALE_SMEM>(g)));
        if (status != IOMB_OK) return status;
    }
    return IOMB_OK;
}

int prepare_rmsnorm_kernels() {
    int status = prepare_family<2, false, false>();
    if (status == IOMB_OK) status = prepare_family<2, false, true>();
    if (status == IOMB_OK) status = prepare_family<2, true, false>();
    if (status == IOMB_OK) status = prepare_family<2, true, true>();
    if (status == IOMB_OK) status = prepare_family<4, false, false>();
    if (status == IOMB_OK) status = prepare_family<4, false, true>();
    if (status == IOMB_OK) status = prepare_family<4, true, false>();
    if (status == IOMB_OK) status = prepare_family<4, true, true>();
    return status;
}

static int rms_dispatch(const iomb_view* x, const iomb_view* residual, const iomb_view* scale,
                        const iomb_view* sum, const iomb_view* out, float eps, int order,
                        void* stream) {
    const bool fused = residual != nullptr;
    ViewFacts fx{}, fs{}, fo{}, fr{}, fm{};
    int status = check_view(x, "rmsnorm x", &fx);
    if (status == IOMB_OK) status = check_view(scale, "rmsnorm scale", &fs);
    if (status == IOMB_OK) status = check_view(out, "rmsnorm out", &fo);
    if (status == IOMB_OK && fused) status = check_view(residual, "add_rmsnorm residual", &fr);
    if (status == IOMB_OK && fused) status = check_view(sum, "add_rmsnorm sum", &fm);
    if (status != IOMB_OK) return status;
    auto same_shape = [](const iomb_view& a, const iomb_view& b) {
        if (a.rank != b.rank) return false;
        for (uint32_t i = 0; i < a.rank; ++i) {
            if (a.dims[i] != b.dims[i]) return false;
        }
        return true;
    };
    // Admission order of validate_rmsnorm (src/device_ops_rmsnorm.cpp:75-127).
    if (!same_shape(*x, *out) || (fused && (!same_shape(*x, *residual) || !same_shape(*x, *sum)))) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rmsnorm x and out shapes differ");
    }
    if (scale->rank != 2 || fs.rows != 1 || fs.cols != fx.cols) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rmsnorm scale must be [1,F]");
    }
    if (x->dtype != out->dtype || x->dtype != scale->dtype
            || (fused && (x->dtype != residual->dtype || x->dtype != sum->dtype))) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rmsnorm data types differ");
    }
    if (out->base == x->base || out->base == scale->base
            || (fused && (out->base == residual->base || out->base == sum->base))) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rmsnorm output must not share an input owner");
    }
    if (fused) {
        if (sum->base == scale->base) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "add_rmsnorm sum must not share the scale owner");
        }
        if ((sum->base == x->base && !same_window(*sum, *x))
                || (sum->base == residual->base && !same_window(*sum, *residual))) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "add_rmsnorm sum alias must be exact");
        }
    }
    if (!(eps >= 0.0f) || eps > 3.402823466e+38f) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rmsnorm epsilon must be finite and nonnegative");
    }
    if (order != IOMB_RMS_LANES16 && order != IOMB_RMS_SEQUENTIAL) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rmsnorm: unknown accumulation order");
    }
    if (x->dtype != IOMB_BF16 && x->dtype != IOMB_F32) {
        return fail(IOMB_ERR_UNSUPPORTED, "rmsnorm: leaf is not BF16 or F32");
    }
    if (fx.rows > 0xFFFFFFFFull || fx.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "rmsnorm: matrix extent exceeds the kernel limit");
    }
    const uint32_t elem = fx.bytes;
    const uint64_t row_bytes = fx.tile_cols * kTile * elem;   // one row of a band
    RmsParams p{};
    const iomb_view* views[4] = {x, out, residual, sum};
    uint64_t strides[4][kMaxLead] = {};
    const uint32_t count = fused ? 4 : 2;
    for (uint32_t k = 0; k < count; ++k) {
        for (uint32_t axis = 0; axis < fx.leading; ++axis) {
            strides[k][axis] = views[k]->plane_strides[axis];
        }
    }
    collapse_leading(fx.leading, x->dims, strides, count, &p.leading);
    p.x = make_operand(*x, fx, strides[0], p.leading, false, false);
    p.out = make_operand(*out, fo, strides[1], p.leading, false, false);
    if (fused) {
        p.residual = make_operand(*residual, fr, strides[2], p.leading, false, false);
        p.sum = make_operand(*sum, fm, strides[3], p.leading, false, false);
    }
    p.scale_row = static_cast<const unsigned char*>(scale->base) + scale->plane_offset * fs.plane_bytes;
    p.rows = static_cast<uint32_t>(fx.rows);
    p.cols = static_cast<uint32_t>(fx.cols);
    p.tile_rows = static_cast<uint32_t>(fx.tile_rows);
    p.tile_cols = static_cast<uint32_t>(fx.tile_cols);
    p.eps = eps;
    p.order = static_cast<uint32_t>(order);
    // Rows of more than 2048 values in the lane order take the pipelined kernel.
    if (order == IOMB_RMS_LANES16 && fx.tile_cols > 128) {
        bool launched = false;
        const int status = launch_rmsnorm_long(p, elem, fused, row_bytes, p.leading.planes * p.tile_rows,
                                               x->storage_bytes, fused ? residual->storage_bytes : 0,
                                               static_cast<cudaStream_t>(stream), &launched);
        if (launched || status != IOMB_OK) return status;
    }
    // Rows per unit: the staged rows (of x, and of the residual when fused) must
    // fit the staging capacity. (Prefetching the next unit into a second buffer
    // was measured 5-25 % slower: the units halve.) The widened
    // scale row joins them in shared memory when three CTAs still fit one SM;
    // otherwise it is read through L1.
    const uint32_t operands = fused ? 2 : 1;
    uint32_t g = kTile;
    while (g > 1 && static_cast<uint64_t>(operands) * g * row_bytes > kUnitCapBytes) g /= 2;
    // Rows so long that the fused form could stage fewer than four of them per operand
    // (tile pieces below a 128-byte line): the addition runs as its own streaming launch
    // and the unfused kernel, with twice the rows per unit, follows on the same stream.
    // Measured at 8192 BF16 features: 510 us for the pair against 594 us fused. The
    // results are the same bits (the fused form stores the rounded sum and normalises it).
    if (fused && static_cast<uint64_t>(g) * kTile * elem < 128) {
        const int added = iomb_binary(IOMB_ADD, x, residual, sum, stream);
        if (added != IOMB_OK) return added;
        return rms_dispatch(sum, nullptr, scale, nullptr, out, eps, order, stream);
    }
    // Long lane chains (256 tiles and more) are hidden better by twice as many, half as
    // large CTAs, as long as a unit's piece of a tile stays a whole 128-byte line
    // (measured: +15 % at 4096 BF16 features, +10 % at 4096 F32; narrower pieces,
    // the fused form and the sequential order all lose).
    if (!fused && order == IOMB_RMS_LANES16 && fx.tile_cols >= 256 && g > 1
            && static_cast<uint64_t>(g / 2) * kTile * elem >= 128) {
        g /= 2;
    }
    // Few rows (decode steps): smaller groups spread the bands over more CTAs; the
    // per-row work is the same, the per-CTA copy shrinks.
    {
        const uint64_t bands = fx.tile_rows * fx.planes;
        const uint64_t wanted = 2 * static_cast<uint64_t>(sm_count() > 0 ? sm_count() : 148);
        while (g > 1 && bands * (kTile / g) < wanted) g /= 2;
    }
    const uint64_t staged_bytes = static_cast<uint64_t>(operands) * g * row_bytes;
    if (staged_bytes > 160 * 1024) {
        // A single row beyond the staging capacity (more than 81 920 BF16 or 40 960 F32
        // values): the unstaged kernel, one CTA per row, both passes from global memory.
        // g == 1 here, so the fused form has already been split into add + rmsnorm above.
        p.group_rows = 1;
        p.groups_per_band = kTile;
        p.units = p.leading.planes * p.tile_rows * kTile;
        const unsigned rows_grid = grid_for(p.units, 8);
        if (elem == 2) rmsnorm_unstaged_kernel<2><<<rows_grid, kRmsThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
        else rmsnorm_unstaged_kernel<4><<<rows_grid, kRmsThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
        return check_launch("rmsnorm launch");
    }
    const uint64_t fixed_bytes = (kTile * kTile + 2 * kTile) * sizeof(float);
    const uint64_t scale_bytes = fx.tile_cols * kTile * sizeof(float);
    const uint64_t per_cta_budget = (227 * 1024) / 3 - 1024;
    const bool scale_smem = staged_bytes + scale_bytes + fixed_bytes <= per_cta_budget;
    const uint64_t smem_bytes = staged_bytes + (scale_smem ? scale_bytes : 0) + fixed_bytes;

    p.group_rows = g;
    p.groups_per_band = kTile / g;
    p.units = p.leading.planes * p.tile_rows * p.groups_per_band;

    RmsKernel kernel = elem == 2 ? pick_kernel<2>(g, fused, scale_smem)
                                 : pick_kernel<4>(g, fused, scale_smem);
    const int prepared = allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
    if (prepared != IOMB_OK) return prepared;
    // Persistent CTAs, as many per SM as shared memory allows: the scale row is
    // staged once per CTA and a CTA's phases overlap with its neighbours'.
    unsigned per_sm = static_cast<unsigned>((227 * 1024) / (smem_bytes + 1024));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    // Short rows (the scale row is at most 2048 values): one CTA per unit in launch
    // order, measured 5-10 % faster than persistent CTAs because the hardware
    // scheduler keeps neighbouring bands together; the per-CTA scale staging hides
    // behind the unit's copies. Long rows: persistent CTAs, so the scale row is
    // scanned once per CTA rather than once per unit.
    const bool one_shot = fx.cols <= 2048;
    const unsigned grid = one_shot ? grid_one_shot(p.units) : grid_for(p.units, per_sm);
    kernel<<<grid, kRmsThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(p);
    char text[160];
    snprintf(text, sizeof text, "rmsnorm_kernel<elem %u, rows %u, %s, scale %s> %s order, %u CTAs x %d",
             elem, g, fused ? "fused" : "unfused", scale_smem ? "in shared memory" : "through L1",
             order == IOMB_RMS_LANES16 ? "lane" : "sequential", grid, kRmsThreads);
    note_launch(text);
    return check_launch("rmsnorm launch");
}

}  // namespace iomb

extern "C" int iomb_rmsnorm(const iomb_view* x, const iomb_view* scale, const iomb_view* out,
                            float eps, int order, void* stream) {
    return iomb::rms_dispatch(x, nullptr, scale, nullptr, out, eps, order, stream);
}

extern "C" int iomb_add_rmsnorm(const iomb_view* x, const iomb_view* residual,
                                const iomb_view* scale, const iomb_view* sum,
                                const iomb_view* out, float eps, int order, void* stream) {
    if (residual == nullptr || sum == nullptr) {
        return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "add_rmsnorm: residual and sum are required");
    }
    return iomb::rms_dispatch(x, residual, scale, sum, out, eps, order, stream);
}


