// RMS normalization of rows longer than 2048 values (optionally fused with the
// preceding residual ADD), lane order.
//
// Replaces standard_tiled_rmsnorm_kernel (src/shared/standard_tiled_rmsnorm.inl:437-637)
// where a 16-row band no longer fits shared memory (8192 BF16 features: 256 KiB).
// Rows are independent, so the unit of work is G rows of one band (G * 32 or G * 64
// contiguous bytes of every tile of the band) sized so that three units fit one SM.
// One persistent CTA of 1024 threads per SM keeps a ring of unit slots in shared memory:
//
//   unfused   slot k % S holds unit k. In iteration k the copies of unit k + S - 2 are
//             started, the chain warps (one thread per row and tile column, 16 * G
//             threads) run the 16 column accumulators of unit k through its tiles in
//             order, and the other warps normalise unit k - 1 and store it. A unit is
//             read from HBM once; the row reduction of one unit hides behind the
//             stores of the previous one and the copies of the next.
//   fused     two slots for x (which becomes the rounded sum in place) and one for the
//             residual. Per unit: add (all threads; the sum is stored), start the next
//             residual copy, chain, normalise (all threads), start the copy of x two
//             units ahead. The phases are serial, the copies are not: x of the next
//             unit and the next residual are in flight the whole time.
//
// Accumulation order (src/cpu/avx512_bf16_rmsnorm_reduction.cpp:69-81,130-148): per
// row 16 column accumulators, each acc = acc + fl(x * x) over the tiles in order, then
// the fixed tree. Bit-identical to rmsnorm.cu's lane order.
#include "rmsnorm.cuh"

#include <stdlib.h>

#include <type_traits>

namespace iomb {

constexpr int kLongThreads = 1024;
constexpr uint32_t kSharedCap = 227 * 1024;
// lanes (256 floats) + two sets of 16 inverses and 16 flags + one flag word, rounded up
constexpr uint32_t kLongFixedBytes = 256 * 4 + 2 * 16 * 4 + 2 * 16 * 4 + 32;

struct LongShape {
    uint32_t slots;           // unfused: ring depth (3 or 4); fused: 3 (x, x, residual)
    uint32_t scale_in_smem;   // the scale row, widened to FP32, is kept in shared memory
    uint32_t debug;           // TEMP measurement switches
};

template <int ELEM, int G, bool FUSED>
__global__ void __launch_bounds__(kLongThreads, 1)
rmsnorm_long_kernel(const RmsParams p, const LongShape shape) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kRowBytes = kTile * ELEM;             // one in-tile row
    constexpr uint32_t kVectorsPerRow = kRowBytes / 16;      // 2 (16-bit) or 4 (32-bit)
    constexpr uint32_t kPerVector = 16 / ELEM;
    constexpr uint32_t kPieceBytes = G * kRowBytes;          // a unit's part of one tile
    constexpr uint32_t kPieceVectors = G * kVectorsPerRow;   // 2 .. 64
    constexpr uint32_t kChains = G * kTile;                  // (row, tile column) pairs
    constexpr uint32_t kChainWarps = (kChains + 31) / 32;
    constexpr uint32_t kChainThreads = kChainWarps * 32;
    // Threads that move vectors: all of them when fused, the warps that do not chain otherwise.
    constexpr uint32_t kMovers = FUSED ? kLongThreads : kLongThreads - kChainThreads;
    static_assert(kLongThreads % kPieceVectors == 0 && kMovers % kPieceVectors == 0,
                  "a thread keeps one vector position of every tile it touches");
    constexpr uint32_t kCopyTilesPerStep = kLongThreads / kPieceVectors;
    constexpr uint32_t kMoveTilesPerStep = kMovers / kPieceVectors;

    const uint32_t unit_bytes = p.tile_cols * kPieceBytes;
    unsigned char* scale_raw = smem + static_cast<size_t>(shape.slots) * unit_bytes;
    float* lanes = reinterpret_cast<float*>(
            scale_raw + (shape.scale_in_smem ? static_cast<size_t>(p.tile_cols) * kTile * 4 : 0));
    float* inverse = lanes + 256;                            // [2][16]
    uint32_t* clean = reinterpret_cast<uint32_t*>(inverse + 32);   // [2][16]
    uint32_t* scale_not_finite = clean + 32;
    const uint32_t tid = threadIdx.x;
    const uint32_t full_tiles = p.cols / kTile;
    const uint32_t tail_cols = p.cols % kTile;

    // Units of this CTA: blockIdx.x, + gridDim.x, ... (neighbouring groups of a band run
    // on neighbouring SMs at the same time).
    const uint32_t count = blockIdx.x < p.units
            ? static_cast<uint32_t>((p.units - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    auto unit_of = [&](uint32_t k) {
        return static_cast<uint64_t>(blockIdx.x) + static_cast<uint64_t>(k) * gridDim.x;
    };

    // Starts the asynchronous copies of one operand's unit k into `slot` (all threads).
    const uint32_t copy_v = tid % kPieceVectors;
    const uint32_t copy_tile0 = tid / kPieceVectors;
    auto issue = [&](const Operand& operand, uint32_t k, unsigned char* slot) {
        if (k >= count || (shape.debug & 4u)) return;
        const RmsUnit at = rms_locate<G>(p, unit_of(k));
        if (!at.valid) return;
        const unsigned char* source = rms_unit_base<ELEM>(p, operand, at) + copy_v * 16;
        unsigned char* target = slot + copy_v * 16;
        for (uint32_t tile = copy_tile0; tile < p.tile_cols; tile += kCopyTilesPerStep) {
            cp_async_16(target + static_cast<size_t>(tile) * kPieceBytes,
                        source + static_cast<size_t>(tile) * kTileBytes);
        }
    };

    // Row sums of squares of the unit in `slot`, then the rows' inverses (chain warps).
    auto chain = [&](uint32_t k, const unsigned char* slot, uint32_t parity, bool scale_finite) {
        const RmsUnit at = rms_locate<G>(p, unit_of(k));
        if (!at.valid) return;                               // uniform per CTA
        const bool active = tid < kChains;
        const uint32_t c = active ? tid : 0;
        const unsigned char* cursor = slot + c * ELEM;       // (row * 16 + lane) * ELEM
        float acc = 0.0f;
        constexpr uint32_t kBatch = 16;
        uint32_t tile = 0;
        if (shape.debug & 1u) { acc = 1.0f; tile = full_tiles; }
        // Squares of sixteen tiles at a time in two register sets: while one set runs
        // through the dependent additions, the loads and products of the other are
        // already issued (a lane is one add every four cycles at best, a load from
        // shared memory takes about thirty).
        auto fetch = [&](float* squares, uint32_t first) {
            const unsigned char* from = cursor + static_cast<size_t>(first) * kPieceBytes;
#pragma unroll
            for (uint32_t j = 0; j < kBatch; ++j) {
                const float value = decode_element<ELEM>(from + j * kPieceBytes);
                squares[j] = __fmul_rn(value, value);
            }
        };
        auto fold = [&](const float* squares) {
#pragma unroll
            for (uint32_t j = 0; j < kBatch; ++j) acc = __fadd_rn(acc, squares[j]);
        };
        if (tile + kBatch <= full_tiles) {
            float even[kBatch], odd[kBatch];
            fetch(even, tile);
            for (;;) {
                // even holds tiles [tile, tile + 16)
                if (tile + 2 * kBatch > full_tiles) { fold(even); tile += kBatch; break; }
                fetch(odd, tile + kBatch);
                fold(even);
                tile += kBatch;
                if (tile + 2 * kBatch > full_tiles) { fold(odd); tile += kBatch; break; }
                fetch(even, tile + kBatch);
                fold(odd);
                tile += kBatch;
            }
        }
        for (; tile < full_tiles; ++tile) {
            acc = accumulate_square(
                    acc, decode_element<ELEM>(cursor + static_cast<size_t>(tile) * kPieceBytes));
        }
        if ((c % kTile) < tail_cols) {
            acc = accumulate_square(
                    acc, decode_element<ELEM>(cursor + static_cast<size_t>(full_tiles) * kPieceBytes));
        }
        if (active) lanes[c] = acc;
        __syncwarp();
        if (active && (c % kTile) == 0) {
            const uint32_t row = c / kTile;
            const float sum = combine_lanes(lanes + row * kTile);
            inverse[parity * 16 + row] = row_inverse(sum, p.cols, p.eps);
            clean[parity * 16 + row] = row_is_clean(sum, scale_finite) ? 1u : 0u;
        }
    };

    // Normalises the unit in `slot` and stores it (mover threads; `m` is the thread's
    // index among them). A thread keeps its vector position (row, column group) and walks
    // tiles m / kPieceVectors, + kMoveTilesPerStep, ...: every address advances by a
    // constant, the row's inverse and its NaN rule are fixed for the whole walk.
    auto emit = [&](uint32_t k, const unsigned char* slot, uint32_t parity, uint32_t m) {
        const RmsUnit at = rms_locate<G>(p, unit_of(k));
        if (!at.valid || (shape.debug & 2u)) return;
        const uint32_t v = m % kPieceVectors;
        const uint32_t row = v / kVectorsPerRow;
        const uint32_t cv = v % kVectorsPerRow;
        const uint32_t live_rows = min(static_cast<uint32_t>(G), at.rows_in_band - at.row0);
        if (row >= live_rows) return;
        const uint32_t col_in_tile = cv * kPerVector;
        const uint32_t first_tile = m / kPieceVectors;
        const float inv = inverse[parity * 16 + row];
        const bool fast = clean[parity * 16 + row] != 0;
        unsigned char* out = rms_unit_base<ELEM>(p, p.out, at) + v * 16
                + static_cast<size_t>(first_tile) * kTileBytes;
        const unsigned char* in = slot + static_cast<size_t>(m) * 16;
        // Whole tiles this thread owns.
        const uint32_t steps = first_tile < full_tiles
                ? (full_tiles - first_tile + kMoveTilesPerStep - 1) / kMoveTilesPerStep : 0;
        auto walk = [&](auto wide_tag, auto fast_tag) {
            constexpr bool kWide = decltype(wide_tag)::value;
            constexpr bool kFast = decltype(fast_tag)::value;
            const unsigned char* w_cursor = kWide
                    ? scale_raw + (static_cast<size_t>(first_tile) * kTile + col_in_tile) * 4
                    : p.scale_row + static_cast<size_t>(first_tile) * kTileBytes + cv * 16;
            constexpr size_t kScaleStep = kWide ? static_cast<size_t>(kMoveTilesPerStep) * kTile * 4
                                                : static_cast<size_t>(kMoveTilesPerStep) * kTileBytes;
            auto load_scale = [&](float* w) {
                if constexpr (kWide) {
                    const float4 w0 = reinterpret_cast<const float4*>(w_cursor)[0];
                    w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
                    if constexpr (ELEM == 2) {
                        const float4 w1 = reinterpret_cast<const float4*>(w_cursor)[1];
                        w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
                    }
                } else {
                    widen_vector<ELEM>(__ldg(reinterpret_cast<const uint4*>(w_cursor)), w);
                }
            };
#pragma unroll 2
            for (uint32_t step = 0; step < steps; ++step) {
                float w[kPerVector];
                load_scale(w);
                store_u4_stream(out, normalize_vector<ELEM>(*reinterpret_cast<const uint4*>(in), w,
                                                            inv, kFast));
                in += static_cast<size_t>(kMoveTilesPerStep) * kPieceBytes;
                out += static_cast<size_t>(kMoveTilesPerStep) * kTileBytes;
                w_cursor += kScaleStep;
            }
            // The ragged last tile, for the thread whose walk reaches it.
            if (tail_cols > col_in_tile && first_tile + steps * kMoveTilesPerStep == full_tiles) {
                float w[kPerVector];
                load_scale(w);
                store_vector_masked<ELEM>(
                        out, normalize_vector<ELEM>(*reinterpret_cast<const uint4*>(in), w, inv, kFast),
                        min(kPerVector, tail_cols - col_in_tile));
            }
        };
        using yes = std::true_type;
        using no = std::false_type;
        if (shape.scale_in_smem) {
            if (fast) walk(yes{}, yes{}); else walk(yes{}, no{});
        } else {
            if (fast) walk(no{}, yes{}); else walk(no{}, no{});
        }
    };

    // ---- prologue: first copies, then the scale row ---------------------------
    unsigned char* const slot0 = smem;
    if constexpr (FUSED) {
        issue(p.x, 0, slot0);
        issue(p.residual, 0, slot0 + 2 * static_cast<size_t>(unit_bytes));
        cp_async_commit();
        issue(p.x, 1, slot0 + unit_bytes);
        cp_async_commit();
    } else {
        for (uint32_t k = 0; k + 2 < shape.slots; ++k) {
            issue(p.x, k, slot0 + static_cast<size_t>(k) * unit_bytes);
            cp_async_commit();
        }
    }
    if (tid == 0) *scale_not_finite = 0;
    __syncthreads();
    for (uint32_t k = tid; k < p.tile_cols * kVectorsPerRow; k += kLongThreads) {
        const uint32_t tile = k / kVectorsPerRow, part = k % kVectorsPerRow;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
                p.scale_row + static_cast<size_t>(tile) * kTileBytes + part * 16));
        float w[kPerVector];
        widen_vector<ELEM>(raw, w);
        const uint32_t first = tile * kTile + part * kPerVector;
        bool finite = true;
#pragma unroll
        for (uint32_t e = 0; e < kPerVector; ++e) {
            // Padding columns of the last tile are not part of the scale.
            if (first + e < p.cols && !(fabsf(w[e]) <= 3.402823466e+38f)) finite = false;
        }
        if (shape.scale_in_smem) {
            float4* wide = reinterpret_cast<float4*>(scale_raw + static_cast<size_t>(first) * 4);
            wide[0] = make_float4(w[0], w[1], w[2], w[3]);
            if constexpr (ELEM == 2) wide[1] = make_float4(w[4], w[5], w[6], w[7]);
        }
        if (!finite) *scale_not_finite = 1;
    }
    __syncthreads();
    const bool scale_finite = *scale_not_finite == 0;

    if constexpr (!FUSED) {
        // Iteration k: unit k is chained while unit k - 1 is normalised and stored; the
        // slot unit k - 2 left is refilled with unit k + S - 2.
        const uint32_t S = shape.slots;
        for (uint32_t k = 0; k <= count; ++k) {
            // Groups committed so far: units 0 .. k + S - 3; unit k must have landed.
            if (S == 3) cp_async_wait<0>(); else cp_async_wait<1>();
            __syncthreads();
            issue(p.x, k + S - 2, slot0 + static_cast<size_t>((k + S - 2) % S) * unit_bytes);
            cp_async_commit();
            if (tid < kChainThreads) {
                if (k < count) chain(k, slot0 + static_cast<size_t>(k % S) * unit_bytes, k & 1u, scale_finite);
            } else if (k >= 1) {
                emit(k - 1, slot0 + static_cast<size_t>((k - 1) % S) * unit_bytes, (k - 1) & 1u,
                     tid - kChainThreads);
            }
        }
    } else {
        unsigned char* const residual_slot = slot0 + 2 * static_cast<size_t>(unit_bytes);
        for (uint32_t k = 0; k < count; ++k) {
            unsigned char* const slot = slot0 + static_cast<size_t>(k & 1u) * unit_bytes;
            // In flight besides x(k), r(k): x(k + 1), the newest group.
            cp_async_wait<1>();
            __syncthreads();
            const RmsUnit at = rms_locate<G>(p, unit_of(k));
            if (at.valid) {
                // sum = x + residual, rounded to the leaf, kept in the slot and stored.
                const uint32_t v = copy_v;
                const uint32_t row = v / kVectorsPerRow;
                const uint32_t col_in_tile = (v % kVectorsPerRow) * kPerVector;
                const bool row_live = row < min(static_cast<uint32_t>(G), at.rows_in_band - at.row0);
                unsigned char* cell = slot + static_cast<size_t>(tid) * 16;
                const unsigned char* other = residual_slot + static_cast<size_t>(tid) * 16;
                unsigned char* sum_out = rms_unit_base<ELEM>(p, p.sum, at) + v * 16
                        + static_cast<size_t>(copy_tile0) * kTileBytes;
                const uint32_t steps = copy_tile0 < full_tiles
                        ? (full_tiles - copy_tile0 + kCopyTilesPerStep - 1) / kCopyTilesPerStep : 0;
#pragma unroll 2
                for (uint32_t step = 0; step < steps; ++step) {
                    const uint4 total = add_vectors<ELEM>(*reinterpret_cast<const uint4*>(cell),
                                                          *reinterpret_cast<const uint4*>(other));
                    *reinterpret_cast<uint4*>(cell) = total;
                    if (row_live) store_u4_stream(sum_out, total);
                    cell += static_cast<size_t>(kCopyTilesPerStep) * kPieceBytes;
                    other += static_cast<size_t>(kCopyTilesPerStep) * kPieceBytes;
                    sum_out += static_cast<size_t>(kCopyTilesPerStep) * kTileBytes;
                }
                if (tail_cols != 0 && copy_tile0 + steps * kCopyTilesPerStep == full_tiles) {
                    const uint4 total = add_vectors<ELEM>(*reinterpret_cast<const uint4*>(cell),
                                                          *reinterpret_cast<const uint4*>(other));
                    *reinterpret_cast<uint4*>(cell) = total;
                    if (row_live && tail_cols > col_in_tile) {
                        store_vector_masked<ELEM>(sum_out, total, min(kPerVector, tail_cols - col_in_tile));
                    }
                }
            }
            __syncthreads();
            issue(p.residual, k + 1, residual_slot);
            cp_async_commit();
            if (tid < kChainThreads) chain(k, slot, 0, scale_finite);
            __syncthreads();
            emit(k, slot, 0, tid);
            __syncthreads();
            issue(p.x, k + 2, slot);
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
}

using LongKernel = void (*)(const RmsParams, const LongShape);

template <int ELEM, bool FUSED>
static LongKernel pick_long(uint32_t g) {
    switch (g) {
        case 16: return rmsnorm_long_kernel<ELEM, 16, FUSED>;
        case 8: return rmsnorm_long_kernel<ELEM, 8, FUSED>;
        case 4: return rmsnorm_long_kernel<ELEM, 4, FUSED>;
        case 2: return rmsnorm_long_kernel<ELEM, 2, FUSED>;
        default: return rmsnorm_long_kernel<ELEM, 1, FUSED>;
    }
}

int prepare_rmsnorm_long_kernels() {
    for (uint32_t g = 1; g <= kTile; g *= 2) {
        const LongKernel kernels[4] = {pick_long<2, false>(g), pick_long<2, true>(g),
                                       pick_long<4, false>(g), pick_long<4, true>(g)};
        for (const LongKernel kernel : kernels) {
            const int status = allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
            if (status != IOMB_OK) return status;
        }
    }
    return IOMB_OK;
}

int launch_rmsnorm_long(const RmsParams& base, uint32_t elem, bool fused, uint64_t row_bytes,
                        uint64_t bands, cudaStream_t stream, bool* launched) {
    *launched = false;
    // Largest group of rows of which three units (and the fixed part) fit one SM.
    const uint64_t room = kSharedCap - kLongFixedBytes;
    if (3 * row_bytes > room) return IOMB_OK;              // not served here
    uint32_t g = kTile;
    while (g > 1 && 3 * g * row_bytes > room) g /= 2;
    // Few rows (decode steps): smaller groups spread the bands over more SMs.
    const uint64_t sms = static_cast<uint64_t>(sm_count() > 0 ? sm_count() : 148);
    while (g > 1 && bands * (kTile / g) < sms) g /= 2;
    const uint64_t unit_bytes = g * row_bytes;
    const uint64_t scale_bytes = row_bytes / elem * 4;     // row 0 of every scale tile as FP32
    LongShape shape{};
    {
        const char* text = getenv("IOMB_RMS_DEBUG");
        shape.debug = text != nullptr ? static_cast<uint32_t>(atoi(text)) : 0;
    }
    shape.slots = 3;
    if (!fused && 4 * unit_bytes + scale_bytes <= room) shape.slots = 4;
    shape.scale_in_smem = shape.slots * unit_bytes + scale_bytes <= room ? 1u : 0u;
    const uint64_t smem_bytes = shape.slots * unit_bytes
            + (shape.scale_in_smem ? scale_bytes : 0) + kLongFixedBytes;

    RmsParams p = base;
    p.group_rows = g;
    p.groups_per_band = kTile / g;
    p.units = bands * p.groups_per_band;
    LongKernel kernel = elem == 2
            ? (fused ? pick_long<2, true>(g) : pick_long<2, false>(g))
            : (fused ? pick_long<4, true>(g) : pick_long<4, false>(g));
    const int prepared = allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
    if (prepared != IOMB_OK) return prepared;
    const uint64_t grid = p.units < sms ? p.units : sms;
    kernel<<<static_cast<unsigned>(grid), kLongThreads, smem_bytes, stream>>>(p, shape);
    *launched = true;
    return check_launch("rmsnorm launch");
}

}  // namespace iomb
