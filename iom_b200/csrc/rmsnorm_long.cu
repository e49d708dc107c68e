// RMS normalization of rows longer than 2048 values (optionally fused with the
// preceding residual ADD), lane order.
//
// Replaces standard_tiled_rmsnorm_kernel (src/shared/standard_tiled_rmsnorm.inl:437-637)
// where a 16-row band no longer fits shared memory (8192 BF16 features: 256 KiB).
// Rows are independent, so the unit of work is G rows of one band (G * 32 or G * 64
// contiguous bytes of every tile of the band) sized so that three units fit one SM.
// One persistent CTA of 512 threads per SM keeps a ring of three unit slots in shared
// memory and, in iteration k, works on three units at once:
//
//   copy     bulk tensor copies bring the next unit into its slot, issued by one thread
//            at the top of the iteration; an mbarrier per slot counts the bytes. Unfused:
//            unit k + 1 of x (three slots). Fused: unit k + 2 of x and of the residual
//            (four slots for x, which becomes the rounded sum in place, two for the
//            residual; the units are half as tall so that the six slots fit).
//   add      fused only: the mover warps add unit k + 1 in its slot and store the sum.
//   chain    the chain warps run the 16 column accumulators of every row of unit k through
//            its tiles in order: a thread owns two neighbouring columns of one row (one
//            32- or 64-bit load per tile, two products, one packed FP32 addition), then the
//            fixed tree and the row's inverse.
//   emit     the mover warps normalise unit k - 1 from its slot and store it.
//
// The chain is the latency-bound part (one dependent addition per tile): its warps sit on
// their own warp schedulers and the movers are the warps of the other schedulers, so the
// chain never waits for an issue slot. One barrier per iteration. A unit is read from HBM
// exactly once; every loop walks with constant strides (no index arithmetic per vector).
//
// Accumulation order (src/cpu/avx512_bf16_rmsnorm_reduction.cpp:69-81,130-148): per
// row 16 column accumulators, each acc = acc + fl(x * x) over the tiles in order, then
// the fixed tree. Bit-identical to rmsnorm.cu's lane order.
#include "rmsnorm.cuh"

#include <cuda.h>

#include <stdio.h>
#include <stdlib.h>

#include <type_traits>

namespace iomb {

constexpr int kLongThreads = 512;
constexpr uint32_t kSharedCap = 227 * 1024;
// pair sums (256 floats) + two sets of 16 inverses and 16 flags + a flag word
constexpr uint32_t kLongFixedBytes = 256 * 4 + 2 * 16 * 4 + 2 * 16 * 4 + 32 + 4 * 8;

struct LongShape {
    uint32_t scale_in_smem;   // the scale row, widened to FP32, is kept in shared memory
    uint32_t scale_in_regs;   // every mover keeps its own scale vectors in registers
    uint32_t box_tiles;       // tiles per bulk copy (the tensor maps' box height)
    uint32_t boxes;           // copies per unit and operand: boxes * box_tiles >= tile_cols
};

// Two FP32 additions in one instruction, each rounded to nearest even (the products that
// feed it are separate scalar multiplications, so nothing can be contracted into an FMA).
__device__ __forceinline__ void add_pair(float& a0, float& a1, float s0, float s1) {
    asm("{\n\t.reg .b64 acc, add;\n\t"
        "mov.b64 acc, {%0, %1};\n\t"
        "mov.b64 add, {%2, %3};\n\t"
        "add.rn.f32x2 acc, acc, add;\n\t"
        "mov.b64 {%0, %1}, acc;\n\t}"
        : "+f"(a0), "+f"(a1) : "f"(s0), "f"(s1));
}

// acc += fl(x * x) for two lanes: one packed multiplication and one packed addition, each
// lane rounded separately exactly like the scalar pair.
__device__ __forceinline__ void square_add_pair(float& a0, float& a1, float x0, float x1) {
    asm("{\n\t.reg .b64 acc, x, sq;\n\t"
        "mov.b64 acc, {%0, %1};\n\t"
        "mov.b64 x, {%2, %3};\n\t"
        "mul.rn.f32x2 sq, x, x;\n\t"
        "add.rn.f32x2 acc, acc, sq;\n\t"
        "mov.b64 {%0, %1}, acc;\n\t}"
        : "+f"(a0), "+f"(a1) : "f"(x0), "f"(x1));
}

// Geometry shared by the kernel and its launcher: chain warps and mover warps of a CTA for
// groups of g rows, and the tiles the movers cover in one step of their walk.
__host__ __device__ constexpr uint32_t long_chain_warps(uint32_t g) { return (g * kTile / 2 + 31) / 32; }
__host__ __device__ constexpr uint32_t long_mover_warps(uint32_t g) {
    return long_chain_warps(g) < 4 ? kLongThreads / 128 * (4 - long_chain_warps(g)) : kLongThreads / 32 - 4;
}
__host__ __device__ constexpr uint32_t long_move_tiles_per_step(uint32_t elem, uint32_t g) {
    return long_mover_warps(g) * 32 / (g * kTile * elem / 16);
}
// A mover keeps the scale vectors of the tiles it walks in registers when its walk has at
// most this many steps (the scale depends on the column only, so one load serves every unit).
constexpr uint32_t kScaleSteps = 12;

// ---- tensor-map copies (TMA) ---------------------------------------------------------
// The unfused kernel fetches a unit with bulk tensor copies: one thread issues them, the
// copy engine generates the addresses and writes shared memory, and an mbarrier counts the
// bytes. No other thread spends an instruction on the copy, and the load/store pipeline
// the chain warps read through stays free of copy instructions.
constexpr uint32_t kMaxBoxTiles = 256;         // a box dimension's limit
constexpr uint32_t kWaitPolls = 1u << 22;      // bounded wait: gives up and reports

__device__ unsigned int g_rms_copy_timeouts;   // counts waits that gave up (never expected)

__device__ __forceinline__ void mbarrier_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(
            static_cast<uint32_t>(__cvta_generic_to_shared(bar))), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarrier_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
            static_cast<uint32_t>(__cvta_generic_to_shared(bar))), "r"(bytes) : "memory");
}
// True when the phase with this parity has completed; polls a bounded number of times.
__device__ __forceinline__ bool mbarrier_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(bar));
    for (uint32_t poll = 0; poll < kWaitPolls; ++poll) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(address), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// One box of the tensor map: coordinates (element in tile, tile column, band of the owner).
__device__ __forceinline__ void tma_load_3d(void* shared_dst, const CUtensorMap* map, uint64_t* bar,
                                            uint32_t c0, uint32_t c1, uint32_t c2) {
    asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst))),
              "l"(reinterpret_cast<uint64_t>(map)),
              "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar))), "r"(c0), "r"(c1), "r"(c2)
            : "memory");
}

// Asks for one box to be brought into L2 (no shared memory, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, uint32_t c0, uint32_t c1, uint32_t c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// Units the L2 prefetch runs ahead of the copy into shared memory: the slots bound how far
// the copies can run ahead (one unit), which leaves HBM idle while a copy's tail lands; the
// prefetch keeps reads in flight across that gap.
#ifndef IOMB_RMS_L2_AHEAD
#define IOMB_RMS_L2_AHEAD 1
#endif

#ifdef IOMB_RMS_TIMING
// Measurement build only: cycles spent per phase by the chain warp and by one mover warp
// of CTA 0 (index 0 wait for copies, 1 barrier, 2 issue, 3 chain, 4 produce, 5 emit, 6 total,
// 7 iterations), chain warp in [0..7], mover warp in [8..15].
__device__ unsigned long long g_rms_timing[16];
#define RMS_TICK(slot)                                                              \
    do {                                                                            \
        if (timing_on) {                                                            \
            const long long now = clock64();                                        \
            atomicAdd(&g_rms_timing[timing_base + (slot)],                          \
                      static_cast<unsigned long long>(now - timing_last));          \
            timing_last = now;                                                      \
        }                                                                           \
    } while (false)
#else
#define RMS_TICK(slot) do {} while (false)
#endif

template <int ELEM, int G, bool FUSED>
__global__ void __launch_bounds__(kLongThreads, 1)
rmsnorm_long_kernel(const RmsParams p, const LongShape shape, const __grid_constant__ CUtensorMap x_map,
                    const __grid_constant__ CUtensorMap r_map) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr uint32_t kSlots = FUSED ? 4 : 3;               // slots of x
    constexpr uint32_t kResidualSlots = FUSED ? 2 : 0;
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kRowBytes = kTile * ELEM;             // one in-tile row
    constexpr uint32_t kVectorsPerRow = kRowBytes / 16;      // 2 (16-bit) or 4 (32-bit)
    constexpr uint32_t kPerVector = 16 / ELEM;
    constexpr uint32_t kPieceBytes = G * kRowBytes;          // a unit's part of one tile
    constexpr uint32_t kPieceVectors = G * kVectorsPerRow;   // 2 .. 64
    constexpr uint32_t kPairs = G * kTile / 2;               // chain threads: (row, column pair)
    constexpr uint32_t kChainWarps = (kPairs + 31) / 32;     // 1, 2 or 4
    constexpr uint32_t kChainThreads = kChainWarps * 32;
    // Warp w issues on scheduler w % 4. The chain warps are warps 0 .. kChainWarps - 1;
    // the movers are the warps of the remaining schedulers (all other warps when every
    // scheduler has a chain warp).
    constexpr uint32_t kFreeSchedulers = kChainWarps < 4 ? 4 - kChainWarps : 0;
    constexpr uint32_t kMoverWarps = long_mover_warps(G);
    constexpr uint32_t kMovers = kMoverWarps * 32;
    static_assert(kMovers % kPieceVectors == 0,
                  "a thread keeps one vector position of every tile it touches");
    constexpr uint32_t kIssuer = 128;                        // warp 4: idle, or the first mover
    constexpr uint32_t kMoveTilesPerStep = kMovers / kPieceVectors;
    static_assert(kChainWarps == long_chain_warps(G) && kMoverWarps == long_mover_warps(G)
                          && kMoveTilesPerStep == long_move_tiles_per_step(ELEM, G),
                  "the launcher sizes the movers' walk with the same geometry");

    // A slot holds whole boxes (the last box of a unit may reach past the row's tiles: the
    // copy engine fills that part with zeros).
    const uint32_t unit_bytes = shape.boxes * shape.box_tiles * kPieceBytes;
    unsigned char* residual_slots = smem + static_cast<size_t>(kSlots) * unit_bytes;
    unsigned char* scale_wide = residual_slots + static_cast<size_t>(kResidualSlots) * unit_bytes;
    float* lanes = reinterpret_cast<float*>(
            scale_wide + (shape.scale_in_smem ? static_cast<size_t>(p.tile_cols) * kTile * 4 : 0));
    float* inverse = lanes + 256;                            // [2][16]
    uint32_t* clean = reinterpret_cast<uint32_t*>(inverse + 32);   // [2][16]
    uint32_t* scale_not_finite = clean + 32;
    uint64_t* full = reinterpret_cast<uint64_t*>(scale_not_finite + 2);   // [kSlots] mbarriers
    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5;
    const uint32_t full_tiles = p.cols / kTile;
    const uint32_t tail_cols = p.cols % kTile;

    uint4 scale_regs[kScaleSteps];                           // movers, when shape.scale_in_regs
    // This thread's index among the movers, or kMovers when it is not one.
    uint32_t mover = kMovers;
    if constexpr (kFreeSchedulers != 0) {
        if ((warp & 3u) >= kChainWarps) {
            mover = ((warp >> 2) * kFreeSchedulers + (warp & 3u) - kChainWarps) * 32 + (tid & 31u);
        }
    } else {
        if (warp >= 4) mover = tid - 128;
    }

    // Units of this CTA: blockIdx.x, + gridDim.x, ... (neighbouring groups of a band run
    // on neighbouring SMs at the same time).
    const uint32_t count = blockIdx.x < p.units
            ? static_cast<uint32_t>((p.units - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    auto unit_of = [&](uint32_t k) {
        return static_cast<uint64_t>(blockIdx.x) + static_cast<uint64_t>(k) * gridDim.x;
    };
    auto slot_of = [&](uint32_t k) { return smem + static_cast<size_t>(k % kSlots) * unit_bytes; };
    auto residual_slot_of = [&](uint32_t k) {
        return residual_slots + static_cast<size_t>(k % (FUSED ? 2 : 1)) * unit_bytes;
    };

    // Starts the copies of unit k into its slot(s): one thread issues the unit's boxes (a
    // copy instruction takes a few hundred cycles to issue: the thread belongs to a warp
    // with no other job whenever the CTA has one, that is unless all four schedulers chain), and asks for a later unit's boxes to be brought into
    // L2. Every unit, valid or not, completes its barrier phase, so the waits stay in step.
    auto issue = [&](uint32_t k) {
        if (tid != kIssuer) return;
        const uint32_t boxes = shape.boxes;
        const uint32_t box_tiles = shape.box_tiles;
        if (k < count) {
            const RmsUnit at = rms_locate<G>(p, unit_of(k));
            uint64_t* bar = full + k % kSlots;
            if (!at.valid) {
                mbarrier_expect_tx(bar, 0);
            } else {
                // The slots were last read and written with ordinary instructions (before
                // the barrier this call follows): order those before the copy engine's writes.
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbarrier_expect_tx(bar, (FUSED ? 2u : 1u) * boxes * box_tiles * kPieceBytes);
                const uint32_t x_band = static_cast<uint32_t>(
                        operand_plane(p.x, p.leading, at.index) * p.x.tile_rows + at.tr);
                unsigned char* target = slot_of(k);
                for (uint32_t box = 0; box < boxes; ++box) {
                    tma_load_3d(target, &x_map, bar, at.row0 * kTile, box * box_tiles, x_band);
                    target += static_cast<size_t>(box_tiles) * kPieceBytes;
                }
                if constexpr (FUSED) {
                    const uint32_t r_band = static_cast<uint32_t>(
                            operand_plane(p.residual, p.leading, at.index) * p.residual.tile_rows + at.tr);
                    target = residual_slot_of(k);
                    for (uint32_t box = 0; box < boxes; ++box) {
                        tma_load_3d(target, &r_map, bar, at.row0 * kTile, box * box_tiles, r_band);
                        target += static_cast<size_t>(box_tiles) * kPieceBytes;
                    }
                }
            }
        }
        if (IOMB_RMS_L2_AHEAD != 0 && k + IOMB_RMS_L2_AHEAD < count) {
            const RmsUnit at = rms_locate<G>(p, unit_of(k + IOMB_RMS_L2_AHEAD));
            if (at.valid) {
                const uint32_t x_band = static_cast<uint32_t>(
                        operand_plane(p.x, p.leading, at.index) * p.x.tile_rows + at.tr);
                for (uint32_t box = 0; box < boxes; ++box) {
                    tma_prefetch_3d(&x_map, at.row0 * kTile, box * box_tiles, x_band);
                }
                if constexpr (FUSED) {
                    const uint32_t r_band = static_cast<uint32_t>(
                            operand_plane(p.residual, p.leading, at.index) * p.residual.tile_rows + at.tr);
                    for (uint32_t box = 0; box < boxes; ++box) {
                        tma_prefetch_3d(&r_map, at.row0 * kTile, box * box_tiles, r_band);
                    }
                }
            }
        }
    };

    // Row sums of squares of unit k, then the rows' inverses (chain warps). Thread c owns
    // columns 2 * (c % 8), + 1 of row c / 8.
    auto chain = [&](uint32_t k, bool scale_finite) {
        const RmsUnit at = rms_locate<G>(p, unit_of(k));
        if (!at.valid) return;                               // uniform per CTA
        const bool active = tid < kPairs;
        const uint32_t c = active ? tid : 0;
        const unsigned char* cursor = slot_of(k) + c * (2 * ELEM);
        float acc0 = 0.0f, acc1 = 0.0f;
        // One load per tile: two BF16 codes in a word, or two floats.
        using Raw = typename std::conditional<ELEM == 2, uint32_t, float2>::type;
        auto squares_of = [&](Raw raw, float& s0, float& s1) {
            float x0, x1;
            if constexpr (ELEM == 2) {
                x0 = bf16_lo(raw);
                x1 = bf16_hi(raw);
            } else {
                x0 = raw.x;
                x1 = raw.y;
            }
            s0 = __fmul_rn(x0, x0);
            s1 = __fmul_rn(x1, x1);
        };
        auto squares = [&](const unsigned char* from, float& s0, float& s1) {
            squares_of(*reinterpret_cast<const Raw*>(from), s0, s1);
        };
        // The raw words of sixteen tiles at a time in two register sets: while one set
        // runs through the dependent additions, the loads of the other are in flight (a
        // lane is one addition every four cycles at best; a load from shared memory takes
        // thirty cycles on an idle SM and several times that while the movers stream).
#ifndef IOMB_RMS_BATCH
#define IOMB_RMS_BATCH 32
#endif
        constexpr uint32_t kBatch = ELEM == 2 ? IOMB_RMS_BATCH : IOMB_RMS_BATCH / 2;
        uint32_t tile = 0;
        auto fetch = [&](Raw* raw, uint32_t first) {
            const unsigned char* from = cursor + static_cast<size_t>(first) * kPieceBytes;
#pragma unroll
            for (uint32_t j = 0; j < kBatch; ++j) {
                raw[j] = *reinterpret_cast<const Raw*>(from + j * kPieceBytes);
            }
        };
        auto fold = [&](const Raw* raw) {
#pragma unroll
            for (uint32_t j = 0; j < kBatch; ++j) {
                if constexpr (ELEM == 2) {
                    square_add_pair(acc0, acc1, bf16_lo(raw[j]), bf16_hi(raw[j]));
                } else {
                    square_add_pair(acc0, acc1, raw[j].x, raw[j].y);
                }
            }
        };
        if (tile + kBatch <= full_tiles) {
            Raw even[kBatch], odd[kBatch];
            fetch(even, tile);
            for (;;) {
                // even holds tiles [tile, tile + kBatch)
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
            float s0, s1;
            squares(cursor + static_cast<size_t>(tile) * kPieceBytes, s0, s1);
            acc0 = __fadd_rn(acc0, s0);
            acc1 = __fadd_rn(acc1, s1);
        }
        if (tail_cols != 0) {
            // The ragged last tile: only its logical columns join the sums.
            float s0, s1;
            squares(cursor + static_cast<size_t>(full_tiles) * kPieceBytes, s0, s1);
            const uint32_t column = 2 * (c % 8);
            if (column < tail_cols) acc0 = __fadd_rn(acc0, s0);
            if (column + 1 < tail_cols) acc1 = __fadd_rn(acc1, s1);
        }
        if (active) {
            lanes[2 * c] = acc0;                             // lanes[row * 16 + column]
            lanes[2 * c + 1] = acc1;
        }
        __syncwarp();
        if (active && (c % 8) == 0) {
            const uint32_t row = c / 8;
            const float sum = combine_lanes(lanes + row * kTile);
            inverse[(k & 1u) * 16 + row] = row_inverse(sum, p.cols, p.eps);
            clean[(k & 1u) * 16 + row] = row_is_clean(sum, scale_finite) ? 1u : 0u;
        }
    };

    // Fused: sum = x + residual for unit k, rounded to the leaf, kept in the x slot and
    // stored (movers). Each mover keeps its vector position and walks tiles first,
    // + kMoveTilesPerStep, ...
    auto add = [&](uint32_t k) {
        if constexpr (FUSED) {
            if (k >= count || mover >= kMovers) return;
            const RmsUnit at = rms_locate<G>(p, unit_of(k));
            if (!at.valid) return;
            const uint32_t v = mover % kPieceVectors;
            const uint32_t row = v / kVectorsPerRow;
            const uint32_t col_in_tile = (v % kVectorsPerRow) * kPerVector;
            const bool row_live = row < min(static_cast<uint32_t>(G), at.rows_in_band - at.row0);
            const uint32_t first_tile = mover / kPieceVectors;
            if (first_tile >= p.tile_cols) return;
            unsigned char* sum = rms_unit_base<ELEM>(p, p.sum, at)
                    + static_cast<size_t>(first_tile) * kTileBytes + v * 16;
            unsigned char* cell = slot_of(k) + static_cast<size_t>(mover) * 16;
            const unsigned char* other = residual_slot_of(k) + static_cast<size_t>(mover) * 16;
            constexpr size_t kGlobalStep = static_cast<size_t>(kMoveTilesPerStep) * kTileBytes;
            constexpr size_t kSlotStep = static_cast<size_t>(kMoveTilesPerStep) * kPieceBytes;
            const uint32_t steps = first_tile < full_tiles
                    ? (full_tiles - first_tile + kMoveTilesPerStep - 1) / kMoveTilesPerStep : 0;
#pragma unroll 2
            for (uint32_t step = 0; step < steps; ++step) {
                const uint4 total = add_vectors<ELEM>(*reinterpret_cast<const uint4*>(cell),
                                                      *reinterpret_cast<const uint4*>(other));
                *reinterpret_cast<uint4*>(cell) = total;
                if (row_live) store_u4_stream(sum, total);
                cell += kSlotStep;
                other += kSlotStep;
                sum += kGlobalStep;
            }
            // The ragged last tile, for the thread whose walk reaches it.
            if (tail_cols != 0 && first_tile + steps * kMoveTilesPerStep == full_tiles) {
                const uint4 total = add_vectors<ELEM>(*reinterpret_cast<const uint4*>(cell),
                                                      *reinterpret_cast<const uint4*>(other));
                *reinterpret_cast<uint4*>(cell) = total;
                if (row_live && tail_cols > col_in_tile) {
                    store_vector_masked<ELEM>(sum, total, min(kPerVector, tail_cols - col_in_tile));
                }
            }
        }
    };

    // Normalises unit k from its slot and stores it (movers).
    auto emit = [&](uint32_t k) {
        if (mover >= kMovers) return;
        const RmsUnit at = rms_locate<G>(p, unit_of(k));
        if (!at.valid) return;
        const uint32_t v = mover % kPieceVectors;
        const uint32_t row = v / kVectorsPerRow;
        const uint32_t cv = v % kVectorsPerRow;
        if (row >= min(static_cast<uint32_t>(G), at.rows_in_band - at.row0)) return;
        const uint32_t col_in_tile = cv * kPerVector;
        const uint32_t first_tile = mover / kPieceVectors;
        const float inv = inverse[(k & 1u) * 16 + row];
        const bool fast = clean[(k & 1u) * 16 + row] != 0;
        unsigned char* out = rms_unit_base<ELEM>(p, p.out, at) + v * 16
                + static_cast<size_t>(first_tile) * kTileBytes;
        const unsigned char* in = slot_of(k) + static_cast<size_t>(mover) * 16;
        const uint32_t steps = first_tile < full_tiles
                ? (full_tiles - first_tile + kMoveTilesPerStep - 1) / kMoveTilesPerStep : 0;
        auto walk = [&](auto wide_tag, auto fast_tag) {
            constexpr bool kWide = decltype(wide_tag)::value;
            constexpr bool kFast = decltype(fast_tag)::value;
            const unsigned char* w_cursor = kWide
                    ? scale_wide + (static_cast<size_t>(first_tile) * kTile + col_in_tile) * 4
                    : p.scale_row + static_cast<size_t>(first_tile) * kTileBytes + cv * 16;
            constexpr size_t kScaleStep = kWide ? static_cast<size_t>(kMoveTilesPerStep) * kTile * 4
                                                : static_cast<size_t>(kMoveTilesPerStep) * kTileBytes;
            auto load_scale = [&](const unsigned char* from, float* w) {
                if constexpr (kWide) {
                    const float4 w0 = reinterpret_cast<const float4*>(from)[0];
                    w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
                    if constexpr (ELEM == 2) {
                        const float4 w1 = reinterpret_cast<const float4*>(from)[1];
                        w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
                    }
                } else {
                    widen_vector<ELEM>(__ldg(reinterpret_cast<const uint4*>(from)), w);
                }
            };
            uint32_t step = 0;
            for (; step + 2 <= steps; step += 2) {
                float w0[kPerVector], w1[kPerVector];
                const uint4 x0 = *reinterpret_cast<const uint4*>(in);
                const uint4 x1 = *reinterpret_cast<const uint4*>(
                        in + static_cast<size_t>(kMoveTilesPerStep) * kPieceBytes);
                load_scale(w_cursor, w0);
                load_scale(w_cursor + kScaleStep, w1);
                store_u4_stream(out, normalize_vector<ELEM>(x0, w0, inv, kFast));
                store_u4_stream(out + static_cast<size_t>(kMoveTilesPerStep) * kTileBytes,
                                normalize_vector<ELEM>(x1, w1, inv, kFast));
                in += 2 * static_cast<size_t>(kMoveTilesPerStep) * kPieceBytes;
                out += 2 * static_cast<size_t>(kMoveTilesPerStep) * kTileBytes;
                w_cursor += 2 * kScaleStep;
            }
            if (step < steps) {
                float w[kPerVector];
                load_scale(w_cursor, w);
                store_u4_stream(out, normalize_vector<ELEM>(*reinterpret_cast<const uint4*>(in), w,
                                                            inv, kFast));
                in += static_cast<size_t>(kMoveTilesPerStep) * kPieceBytes;
                out += static_cast<size_t>(kMoveTilesPerStep) * kTileBytes;
                w_cursor += kScaleStep;
            }
            // The ragged last tile, for the thread whose walk reaches it.
            if (tail_cols > col_in_tile && first_tile + steps * kMoveTilesPerStep == full_tiles) {
                float w[kPerVector];
                load_scale(w_cursor, w);
                store_vector_masked<ELEM>(
                        out, normalize_vector<ELEM>(*reinterpret_cast<const uint4*>(in), w, inv, kFast),
                        min(kPerVector, tail_cols - col_in_tile));
            }
        };
        // The walk with the scale in registers: loads of three steps, then their stores.
        auto walk_regs = [&](auto fast_tag) {
            constexpr bool kFast = decltype(fast_tag)::value;
            constexpr size_t kSlotStep = static_cast<size_t>(kMoveTilesPerStep) * kPieceBytes;
            constexpr size_t kGlobalStep = static_cast<size_t>(kMoveTilesPerStep) * kTileBytes;
#pragma unroll
            for (uint32_t half = 0; half < kScaleSteps; half += 3) {
                uint4 xs[3];
#pragma unroll
                for (uint32_t j = 0; j < 3; ++j) {
                    if (half + j < steps) xs[j] = *reinterpret_cast<const uint4*>(in + (half + j) * kSlotStep);
                }
#pragma unroll
                for (uint32_t j = 0; j < 3; ++j) {
                    if (half + j < steps) {
                        float w[kPerVector];
                        widen_vector<ELEM>(scale_regs[half + j], w);
                        store_u4_stream(out + (half + j) * kGlobalStep,
                                        normalize_vector<ELEM>(xs[j], w, inv, kFast));
                    }
                }
            }
            // The ragged last tile, for the thread whose walk reaches it.
            if (tail_cols > col_in_tile && first_tile + steps * kMoveTilesPerStep == full_tiles) {
                uint4 raw = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (uint32_t j = 0; j < kScaleSteps; ++j) {
                    if (j == steps) raw = scale_regs[j];
                }
                float w[kPerVector];
                widen_vector<ELEM>(raw, w);
                store_vector_masked<ELEM>(
                        out + steps * kGlobalStep,
                        normalize_vector<ELEM>(*reinterpret_cast<const uint4*>(in + steps * kSlotStep),
                                               w, inv, kFast),
                        min(kPerVector, tail_cols - col_in_tile));
            }
        };
        using yes = std::true_type;
        using no = std::false_type;
        if (shape.scale_in_regs) {
            if (fast) walk_regs(yes{}); else walk_regs(no{});
        } else if (shape.scale_in_smem) {
            if (fast) walk(yes{}, yes{}); else walk(yes{}, no{});
        } else {
            if (fast) walk(no{}, yes{}); else walk(no{}, no{});
        }
    };

    // ---- prologue: the first copies, then the scale row ---------------------------
    if (tid == 0) {
        *scale_not_finite = 0;
        for (uint32_t slot = 0; slot < kSlots; ++slot) mbarrier_init(full + slot, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    issue(0);
    if constexpr (FUSED) issue(1);
    for (uint32_t i = tid; i < p.tile_cols * kVectorsPerRow; i += kLongThreads) {
        const uint32_t tile = i / kVectorsPerRow, part = i % kVectorsPerRow;
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
            float4* wide = reinterpret_cast<float4*>(scale_wide + static_cast<size_t>(first) * 4);
            wide[0] = make_float4(w[0], w[1], w[2], w[3]);
            if constexpr (ELEM == 2) wide[1] = make_float4(w[4], w[5], w[6], w[7]);
        }
        if (!finite) *scale_not_finite = 1;
    }
    __syncthreads();
    const bool scale_finite = *scale_not_finite == 0;
    // Iteration k: unit k is chained and unit k - 1 emitted; unfused, unit k + 1 is being
    // copied; fused, unit k + 1 is added and unit k + 2 copied. At the barrier unit k is
    // complete in its slot (the copy, or the sum), the inverses of unit k - 1 are known, and
    // the slot the new copies go to has been emitted (x) or added (residual) in the
    // iteration before.
    //
    // Who reads what the copy engine wrote waits for that unit's mbarrier itself: the chain
    // warps (unfused) before the iteration's barrier, the movers right before they first
    // read the unit (its copy has had an iteration or more by then, so they seldom poll).
    // Warps with neither job only take part in the barriers. A wait that gives up (it never
    // should) makes every thread leave at the next barrier, before anything more is
    // computed from a slot that may be incomplete.
#ifdef IOMB_RMS_TIMING
    const bool timing_on = blockIdx.x == 0 && (tid == 0 || tid == 32);
    const uint32_t timing_base = tid == 0 ? 0 : 8;
    long long timing_last = clock64();
    const long long timing_start = timing_last;
#endif
    bool copies_arrive = true;
    auto landed = [&](uint32_t k) {
        if (k < count && !mbarrier_wait(full + k % kSlots, (k / kSlots) & 1u)) copies_arrive = false;
        return copies_arrive;
    };
    auto meet = [&]() {
        RMS_TICK(0);
        if (__syncthreads_or(!copies_arrive)) {
            if (tid == 0) atomicAdd(&g_rms_copy_timeouts, 1u);
            copies_arrive = false;
            return false;
        }
        RMS_TICK(1);
        return true;
    };
    // The chain warps and the others run loops of their own (the same barriers in the same
    // order), so that neither side's registers count against the other's.
    if (tid < kChainThreads) {
        bool running = true;
        if constexpr (FUSED) running = meet();               // unit 0 has been added
        for (uint32_t k = 0; running && k <= count; ++k) {
            if constexpr (!FUSED) landed(k);
            if (!meet()) break;
            if (k < count) chain(k, scale_finite);
            RMS_TICK(3);
        }
    } else {
        const bool moves = mover < kMovers;
        bool running = true;
#pragma unroll
        for (uint32_t j = 0; j < kScaleSteps; ++j) scale_regs[j] = make_uint4(0, 0, 0, 0);
        if (shape.scale_in_regs && moves) {
            const uint32_t first_tile = mover / kPieceVectors;
            const uint32_t cv = mover % kPieceVectors % kVectorsPerRow;
#pragma unroll
            for (uint32_t j = 0; j < kScaleSteps; ++j) {
                const uint32_t tile = first_tile + j * kMoveTilesPerStep;
                if (tile < p.tile_cols) {
                    scale_regs[j] = __ldg(reinterpret_cast<const uint4*>(
                            p.scale_row + static_cast<size_t>(tile) * kTileBytes + cv * 16));
                }
            }
        }
        if constexpr (FUSED) {
            // Unit 0 is added before the loop: from then on the add runs one unit ahead of
            // the chain.
            if (moves && landed(0)) add(0);
            running = meet();
        }
        for (uint32_t k = 0; running && k <= count; ++k) {
            if (!meet()) break;
            issue(k + (FUSED ? 2 : 1));
            RMS_TICK(2);
            if (moves) {
                if (k >= 1 && (FUSED || landed(k - 1))) emit(k - 1);
                RMS_TICK(5);
                if constexpr (FUSED) {
                    if (landed(k + 1)) add(k + 1);
                }
                RMS_TICK(4);
            }
        }
    }
    // Leaving early with copies possibly in flight: give them a bounded time to land
    // before the CTA's shared memory is handed to another CTA.
    if (!copies_arrive && tid == 0) {
        for (uint32_t slot = 0; slot < kSlots; ++slot) {
            (void)mbarrier_wait(full + slot, 0);
            (void)mbarrier_wait(full + slot, 1);
        }
    }
#ifdef IOMB_RMS_TIMING
    if (timing_on) {
        atomicAdd(&g_rms_timing[timing_base + 6], static_cast<unsigned long long>(clock64() - timing_start));
        atomicAdd(&g_rms_timing[timing_base + 7], static_cast<unsigned long long>(count + 1));
    }
#endif
}

using LongKernel = void (*)(const RmsParams, const LongShape, const CUtensorMap, const CUtensorMap);

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

// cuTensorMapEncodeTiled through the runtime's driver entry point table (the library does
// not link the driver directly). Pure host arithmetic: no allocation, no device work.
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
    static const EncodeTiled entry = [] {
        void* symbol = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &found)
                    != cudaSuccess
                || found != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            return static_cast<EncodeTiled>(nullptr);
        }
        return reinterpret_cast<EncodeTiled>(symbol);
    }();
    return entry;
}

// The owner's storage as (element in tile, tile column, band): a unit's part of a band is
// the box {g * 16 elements, box_tiles tiles, 1 band} at element g-row * 16 of every tile.
static bool make_unit_map(CUtensorMap* map, const Operand& operand, uint64_t storage_bytes,
                          uint32_t elem, uint32_t g, uint32_t box_tiles) {
    const EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const uint64_t tile_bytes = static_cast<uint64_t>(kTileSlots) * elem;
    const uint64_t band_bytes = operand.tile_cols * tile_bytes;
    const cuuint64_t dims[3] = {kTileSlots, operand.tile_cols, storage_bytes / band_bytes};
    const cuuint64_t strides[2] = {tile_bytes, band_bytes};
    const cuuint32_t box[3] = {g * kTile, box_tiles, 1};
    const cuuint32_t element_strides[3] = {1, 1, 1};
    if (dims[2] == 0 || dims[2] > 0x7FFFFFFFull || dims[1] > 0x7FFFFFFFull) return false;   // signed coordinates
    return encode(map, elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 3,
                  operand.base, dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_rmsnorm_long(const RmsParams& base, uint32_t elem, bool fused, uint64_t row_bytes,
                        uint64_t bands, uint64_t x_storage_bytes, uint64_t residual_storage_bytes,
                        cudaStream_t stream, bool* launched) {
    *launched = false;
    // A unit is copied as `boxes` equal boxes of at most kMaxBoxTiles tiles; the slots hold
    // whole boxes. Largest group of rows of which the slots (and the fixed part) fit one SM.
    const uint64_t room = kSharedCap - kLongFixedBytes;
    const uint64_t slots = fused ? 6 : 3;
    const uint32_t boxes = (base.tile_cols + kMaxBoxTiles - 1) / kMaxBoxTiles;
    // (a multiple of four tiles, so that every box starts on a 128-byte boundary of its slot)
    const uint32_t box_tiles = ((base.tile_cols + boxes - 1) / boxes + 3) / 4 * 4;
    const uint64_t slot_row_bytes = static_cast<uint64_t>(boxes) * box_tiles * kTile * elem;
    if (slots * slot_row_bytes > room) return IOMB_OK;     // not served here
    uint32_t g = kTile;
    while (g > 1 && slots * g * slot_row_bytes > room) g /= 2;
    // Few rows (decode steps): smaller groups spread the bands over more SMs.
    const uint64_t sms = static_cast<uint64_t>(sm_count() > 0 ? sm_count() : 148);
    while (g > 1 && bands * (kTile / g) < sms) g /= 2;
    const uint64_t unit_bytes = g * slot_row_bytes;
    const uint64_t scale_bytes = row_bytes / elem * 4;     // row 0 of every scale tile as FP32
    LongShape shape{};
    shape.boxes = boxes;
    shape.box_tiles = box_tiles;
    const uint64_t walk_tiles = long_move_tiles_per_step(elem, g);
    shape.scale_in_regs = (base.tile_cols + walk_tiles - 1) / walk_tiles <= kScaleSteps ? 1u : 0u;
    shape.scale_in_smem = !shape.scale_in_regs && slots * unit_bytes + scale_bytes <= room ? 1u : 0u;
    const uint64_t smem_bytes = slots * unit_bytes + (shape.scale_in_smem ? scale_bytes : 0) + kLongFixedBytes;

    RmsParams p = base;
    p.group_rows = g;
    p.groups_per_band = kTile / g;
    p.units = bands * p.groups_per_band;
    CUtensorMap x_map{}, r_map{};
    if (!make_unit_map(&x_map, p.x, x_storage_bytes, elem, g, box_tiles)
            || (fused && !make_unit_map(&r_map, p.residual, residual_storage_bytes, elem, g, box_tiles))) {
        return IOMB_OK;                                    // no tensor maps here: not served
    }
    LongKernel kernel = elem == 2
            ? (fused ? pick_long<2, true>(g) : pick_long<2, false>(g))
            : (fused ? pick_long<4, true>(g) : pick_long<4, false>(g));
    const int prepared = allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
    if (prepared != IOMB_OK) return prepared;
    const uint64_t grid = p.units < sms ? p.units : sms;
    kernel<<<static_cast<unsigned>(grid), kLongThreads, smem_bytes, stream>>>(p, shape, x_map, r_map);
    *launched = true;
    char text[160];
    snprintf(text, sizeof text, "rmsnorm_long_kernel<elem %u, rows %u, %s> %s, scale %s, %u CTAs x %d",
             elem, g, fused ? "fused" : "unfused", "tensor-map copies",
             shape.scale_in_regs ? "in registers" : shape.scale_in_smem ? "in shared memory" : "through L1", static_cast<unsigned>(grid),
             kLongThreads);
    note_launch(text);
    return check_launch("rmsnorm launch");
}

}  // namespace iomb

#ifdef IOMB_RMS_TIMING
extern "C" int iomb_debug_rms_timing(unsigned long long* out, int reset) {
    if (cudaDeviceSynchronize() != cudaSuccess) return 1;
    if (cudaMemcpyFromSymbol(out, iomb::g_rms_timing, sizeof(unsigned long long) * 16) != cudaSuccess) return 2;
    if (reset) {
        unsigned long long zero[16] = {};
        if (cudaMemcpyToSymbol(iomb::g_rms_timing, zero, sizeof zero) != cudaSuccess) return 3;
    }
    return 0;
}
#endif
