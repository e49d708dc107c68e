// RMS normalization of rows longer than 2048 values (optionally fused with the
// preceding residual ADD), lane order.
//
// Replaces standard_tiled_rmsnorm_kernel (src/shared/standard_tiled_rmsnorm.inl:437-637)
// where a 16-row band no longer fits shared memory (8192 BF16 features: 256 KiB).
// Rows are independent, so the unit of work is G rows of one band (G * 32 or G * 64
// contiguous bytes of every tile of the band). One persistent CTA of 512 threads per SM
// keeps a ring of unit slots in shared memory; its warps have one job each and hand units
// on through mbarriers, so no job waits for another longer than the data demands:
//
//   copy     one thread issues bulk tensor copies (TMA) of the next unit of x (and of the
//            residual) into a free slot, and asks for the unit after it to be brought into
//            L2. An mbarrier per slot counts the bytes that landed.
//   add      fused only: the mover warps add a landed unit in its slot (x becomes the
//            rounded sum in place) and store the sum.
//   chain    a chain warp runs the 16 column accumulators of every row of a unit through
//            its tiles in order: a thread owns two neighbouring columns of one row (one
//            32- or 64-bit load per tile, one packed product, one packed FP32 addition),
//            then the fixed tree and the row's inverse. This is the latency-bound part (one
//            dependent addition per tile, whatever G is). When a unit is so small that one
//            chain no longer keeps up with HBM (G <= 2: long rows, or the fused kernel's
//            half-height units), two or three chain warps take alternate units and each
//            has that many units' time.
//   emit     the mover warps normalise a chained unit from its slot and store it.
//
// With one chain of an unfused kernel, the chain warps sit on warp schedulers of their own
// (warp w issues on scheduler w % 4) and the movers are the warps of the other schedulers;
// fused, where the movers do twice the work, and with several chains, they are all warps but
// the chains' and the issuing thread's. Movers keep their part of the scale row in registers. A unit is read from HBM exactly once; every loop walks with constant strides.
//
// Every wait is bounded: a wait that gives up sets a flag that ends all jobs of the CTA, and
// the launch is counted in a device counter the host can read (iomb_rmsnorm_copy_timeouts).
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

struct LongShape {
    uint32_t scale_in_smem;   // the scale row, widened to FP32, is kept in shared memory
    uint32_t scale_in_regs;   // every mover keeps its own scale vectors in registers
    uint32_t box_tiles;       // tiles per bulk copy (the tensor maps' box height)
    uint32_t boxes;           // copies per unit and operand: boxes * box_tiles >= tile_cols
};

// acc += fl(x * x) for two lanes: two scalar multiplications, each rounded, and one packed
// addition that rounds each lane like the scalar one. The products are not packed: a packed
// product feeding a packed sum is contracted into a fused multiply-add by the assembler
// whatever the rounding qualifiers say (F32 rows then differ from the separately rounded
// recurrence of src/cpu/queue.cpp:1187-1196 in their last bits).
__device__ __forceinline__ void square_add_pair(float& a0, float& a1, float x0, float x1) {
    const float s0 = __fmul_rn(x0, x0);
    const float s1 = __fmul_rn(x1, x1);
    asm("{\n\t.reg .b64 acc, add;\n\t"
        "mov.b64 acc, {%0, %1};\n\t"
        "mov.b64 add, {%2, %3};\n\t"
        "add.rn.f32x2 acc, acc, add;\n\t"
        "mov.b64 {%0, %1}, acc;\n\t}"
        : "+f"(a0), "+f"(a1) : "f"(s0), "f"(s1));
}

// Geometry shared by the kernel and its launcher, for groups of g rows.
// Columns a chain thread owns (one while the chain then still fits two warps: a thread's
// step is then a load, a decode, a product and the dependent addition, the shortest there
// is; two neighbouring columns with packed arithmetic otherwise), and the warps of one chain:
__host__ __device__ constexpr uint32_t long_chain_pack(uint32_t g, bool) { return g <= 4 ? 1 : 2; }
__host__ __device__ constexpr uint32_t long_chain_warps(uint32_t g, bool fused) {
    return (g * kTile / long_chain_pack(g, fused) + 31) / 32;
}
// Chains that run side by side on alternate units: the time of a chain per unit does not
// shrink with g (one dependent addition per tile of the row) while the unit's HBM time does,
// so small groups need several (only chains of one warp are multiplied: g <= 2).
constexpr uint32_t kMaxChains = 3;
// (three chains were measured slower than two for the fused kernel: 0.63 against 0.69 of the
// copy peak at 12288 features, where both fit)
__host__ __device__ constexpr uint32_t long_most_chains(uint32_t g, bool fused) {
    return long_chain_warps(g, fused) == 1 ? (fused ? 2 : kMaxChains) : 1;
}
// Movers, and the tiles they cover in one step of their walk. With one chain of an unfused
// kernel they are the warps of the schedulers without a chain warp (sharing them cost that
// kernel 14 %; all other warps when every scheduler has a chain warp). The fused kernel's
// movers do twice the work per byte (add, then emit: measured +3-4 % on [262144, 8192] and
// [32768, 8192]), and kernels with several chains leave few schedulers free: there the movers
// are all warps but the chains' and the issuing thread's.
__host__ __device__ constexpr bool long_movers_everywhere(bool fused, uint32_t chains) {
    return fused || chains > 1;
}
__host__ __device__ constexpr uint32_t long_mover_warps(uint32_t g, bool fused, uint32_t chains) {
    if (long_movers_everywhere(fused, chains) && long_chain_warps(g, fused) * chains < 4) {
        return kLongThreads / 32 - long_chain_warps(g, fused) * chains - 1;
    }
    return long_chain_warps(g, fused) * chains < 4
            ? kLongThreads / 128 * (4 - long_chain_warps(g, fused) * chains)
            : kLongThreads / 32 - 4;
}
__host__ __device__ constexpr uint32_t long_move_tiles_per_step(uint32_t elem, uint32_t g, bool fused,
                                                                uint32_t chains) {
    return long_mover_warps(g, fused, chains) * 32 / (g * kTile * elem / 16);
}
// Slots of x: a unit holds its slot from the copy (one unit ahead) through the add (fused),
// the chain (one unit's time per chain) and the emit. The residual has two slots of its own.
__host__ __device__ constexpr uint32_t long_x_slots(bool fused, uint32_t chains) {
    return fused ? 3 + chains : 2 + chains;
}
__host__ __device__ constexpr uint32_t long_slots(bool fused, uint32_t chains) {
    return long_x_slots(fused, chains) + (fused ? 2 : 0);
}
// Shared memory besides the slots: the chains' lane sums, per slot 16 inverses and 16
// flags, two flag words, four mbarriers per slot.
__host__ __device__ constexpr uint32_t long_fixed_bytes(uint32_t g, bool fused, uint32_t chains) {
    return chains * g * kTile * 4 + long_x_slots(fused, chains) * (16 * 4 + 16 * 4) + 16
            + long_x_slots(fused, chains) * 4 * 8;
}
// A mover keeps the scale vectors of the tiles it walks in registers when its walk has at
// most this many steps (the scale depends on the column only, so one load serves every unit).
// (Sixteen vectors are 64 registers. The fused kernel's movers also add, and ran 13 % slower
// with that many registers held: they keep eight, which covers 8192 features.)
__host__ __device__ constexpr uint32_t long_scale_steps(bool fused) { return fused ? 8 : 16; }

// ---- tensor-map copies (TMA) and mbarriers ---------------------------------------------
// A unit is fetched with bulk tensor copies: one thread issues them, the copy engine
// generates the addresses and writes shared memory, and an mbarrier counts the bytes. No
// other thread spends an instruction on the copy, and the load/store pipeline the chain
// warps read through stays free of copy instructions.
constexpr uint32_t kMaxBoxTiles = 256;         // a box dimension's limit
constexpr long long kWaitCycles = 1ll << 31;   // bounded wait (about a second): gives up and reports

__device__ unsigned int g_rms_copy_timeouts;   // counts waits that gave up (never expected)

__device__ __forceinline__ void mbarrier_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(
            static_cast<uint32_t>(__cvta_generic_to_shared(bar))), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarrier_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
            static_cast<uint32_t>(__cvta_generic_to_shared(bar))), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(
            static_cast<uint32_t>(__cvta_generic_to_shared(bar))) : "memory");
}
__device__ __forceinline__ bool mbarrier_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar))), "r"(parity)
                 : "memory");
    return done != 0;
}
// True when the phase with this parity has completed. Polls for a bounded time and gives
// up at once when another wait of the CTA has given up (`stop`); a wait that gives up sets
// `stop` itself.
__device__ __forceinline__ bool mbarrier_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* stop) {
    if (mbarrier_test(bar, parity)) return true;
    const long long start = clock64();
    do {
        if (mbarrier_test(bar, parity)) return true;
        if (*stop != 0) return false;
    } while (clock64() - start < kWaitCycles);
    *stop = 1;
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
constexpr uint32_t kL2Ahead = 1;
// Most units a CTA works through in one launch (see launch_rmsnorm_long).
constexpr uint32_t kUnitsPerCtaAndLaunch = 128;

template <int ELEM, int G, bool FUSED, int CHAINS>
__global__ void __launch_bounds__(kLongThreads, 1)
rmsnorm_long_kernel(const RmsParams p, const LongShape shape, const __grid_constant__ CUtensorMap x_map,
                    const __grid_constant__ CUtensorMap r_map) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kRowBytes = kTile * ELEM;             // one in-tile row
    constexpr uint32_t kVectorsPerRow = kRowBytes / 16;      // 2 (16-bit) or 4 (32-bit)
    constexpr uint32_t kPerVector = 16 / ELEM;
    constexpr uint32_t kPieceBytes = G * kRowBytes;          // a unit's part of one tile
    constexpr uint32_t kPieceVectors = G * kVectorsPerRow;   // 2 .. 64
    constexpr uint32_t kScaleSteps = long_scale_steps(FUSED);
    constexpr uint32_t kPack = long_chain_pack(G, FUSED);           // columns per chain thread
    constexpr uint32_t kPairs = G * kTile / kPack;           // threads of a chain
    constexpr uint32_t kChainWarps = long_chain_warps(G, FUSED);    // 1, 2 or 4
    constexpr uint32_t kChains = CHAINS;                     // chains on alternate units
    constexpr uint32_t kChainThreads = kChainWarps * 32;
    constexpr uint32_t kAllChainWarps = kChainWarps * kChains;
    // Warp w issues on scheduler w % 4. The chain warps are warps 0 .. kAllChainWarps - 1;
    // the movers are the warps of the remaining schedulers (unfused) or every other warp
    // but the issuing thread's (fused); all other warps when every scheduler has a chain warp.
    constexpr uint32_t kFreeSchedulers = kAllChainWarps < 4 ? 4 - kAllChainWarps : 0;
    constexpr uint32_t kMoverWarps = long_mover_warps(G, FUSED, CHAINS);
    constexpr uint32_t kMovers = kMoverWarps * 32;
    static_assert(kMovers % kPieceVectors == 0,
                  "a thread keeps one vector position of every tile it touches");
    constexpr uint32_t kIssuer = 128;                        // warp 4: no other job, or the first mover
    constexpr uint32_t kMoveTilesPerStep = long_move_tiles_per_step(ELEM, G, FUSED, CHAINS);
    static_assert(kMoveTilesPerStep == kMovers / kPieceVectors, "the launcher sizes the walk alike");
    // The pipeline, in units: the copy runs kCopyAhead units ahead of the movers' step; the
    // emit follows kLag units behind it (the chains' time, plus the add's when fused).
    constexpr uint32_t kSlots = long_x_slots(FUSED, CHAINS);
    constexpr uint32_t kResidualSlots = FUSED ? 2 : 0;
    constexpr uint32_t kCopyAhead = 1;
    constexpr uint32_t kLag = FUSED ? kChains + 1 : kChains;
    static_assert(kSlots == kCopyAhead + kLag + 1, "a slot is free again when its unit was emitted");

    // A slot holds whole boxes (the last box of a unit may reach past the row's tiles: the
    // copy engine fills that part with zeros).
    const uint32_t unit_bytes = shape.boxes * shape.box_tiles * kPieceBytes;
    unsigned char* residual_slots = smem + static_cast<size_t>(kSlots) * unit_bytes;
    unsigned char* scale_wide = residual_slots + static_cast<size_t>(kResidualSlots) * unit_bytes;
    float* lanes = reinterpret_cast<float*>(
            scale_wide + (shape.scale_in_smem ? static_cast<size_t>(p.tile_cols) * kTile * 4 : 0));
    float* inverse = lanes + kChains * G * kTile;            // [kSlots][16]
    uint32_t* clean = reinterpret_cast<uint32_t*>(inverse + kSlots * 16);   // [kSlots][16]
    uint32_t* scale_not_finite = clean + kSlots * 16;
    volatile uint32_t* stop = scale_not_finite + 1;          // a wait gave up: every job ends
    // Per slot: the copy landed; (fused) the sum is in the slot; the inverses are known; the
    // unit was emitted.
    uint64_t* landed_bar = reinterpret_cast<uint64_t*>(scale_not_finite + 4);
    uint64_t* added_bar = landed_bar + kSlots;
    uint64_t* chained_bar = added_bar + kSlots;
    uint64_t* emitted_bar = chained_bar + kSlots;
    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5;
    const uint32_t lane = tid & 31u;
    const uint32_t full_tiles = p.cols / kTile;
    const uint32_t tail_cols = p.cols % kTile;

    uint4 scale_regs[kScaleSteps];                           // movers, when shape.scale_in_regs
    // This thread's index among the movers, or kMovers when it is not one.
    uint32_t mover = kMovers;
    if constexpr (long_movers_everywhere(FUSED, CHAINS) && kFreeSchedulers != 0) {
        if (warp >= kAllChainWarps && warp != 4) {
            mover = (warp - kAllChainWarps - (warp > 4 ? 1u : 0u)) * 32 + lane;
        }
    } else if constexpr (kFreeSchedulers != 0) {
        if ((warp & 3u) >= kAllChainWarps) {
            mover = ((warp >> 2) * kFreeSchedulers + (warp & 3u) - kAllChainWarps) * 32 + lane;
        }
    } else {
        if (warp >= 4) mover = tid - 128;
    }

    // Units of this CTA: blockIdx.x, + gridDim.x, ... (neighbouring groups of a band run
    // on neighbouring SMs at the same time).
    const uint32_t count = blockIdx.x < p.units
            ? static_cast<uint32_t>((p.units - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    auto unit_of = [&](uint32_t k) {
        return p.first_unit + blockIdx.x + static_cast<uint64_t>(k) * gridDim.x;
    };
    auto slot_of = [&](uint32_t k) { return smem + static_cast<size_t>(k % kSlots) * unit_bytes; };
    auto residual_slot_of = [&](uint32_t k) {
        return residual_slots + static_cast<size_t>(k % (FUSED ? 2 : 1)) * unit_bytes;
    };
    // Unit k's turn on one of the per-slot barriers: slot k % kSlots, phase k / kSlots.
    auto await = [&](uint64_t* bars, uint32_t k) {
        return mbarrier_wait(bars + k % kSlots, (k / kSlots) & 1u, stop);
    };
    // One arrival per warp, after all its lanes' reads and writes of the unit.
    auto warp_arrives = [&](uint64_t* bars, uint32_t k) {
        __syncwarp();
        if (lane == 0) mbarrier_arrive(bars + k % kSlots);
    };

    // Starts the copies of unit k into its slot(s) once those are free, and asks for a
    // later unit's boxes to be brought into L2. One thread does this (a copy instruction
    // takes a few hundred cycles to issue: the thread belongs to a warp with no other job
    // whenever the CTA has one, that is unless all four schedulers chain). Every unit,
    // valid or not, completes its barrier phases, so the waits stay in step.
    auto issue = [&](uint32_t k) {
        if (tid != kIssuer) return true;
        const uint32_t boxes = shape.boxes;
        const uint32_t box_tiles = shape.box_tiles;
        if (k < count) {
            // The slot of x held unit k - kSlots (emitted?), the residual's unit k - 2 (added?).
            if (k >= kSlots && !await(emitted_bar, k - kSlots)) return false;
            if constexpr (FUSED) {
                if (k >= 2 && !await(added_bar, k - 2)) return false;
            }
            const RmsUnit at = rms_locate<G>(p, unit_of(k));
            uint64_t* bar = landed_bar + k % kSlots;
            if (!at.valid) {
                mbarrier_expect_tx(bar, 0);
            } else {
                // The slots were last read and written with ordinary instructions: order
                // those before the copy engine's writes.
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
        if (kL2Ahead != 0 && k + kL2Ahead < count) {
            const RmsUnit at = rms_locate<G>(p, unit_of(k + kL2Ahead));
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
        return true;
    };

    // Row sums of squares of unit k, then the rows' inverses (the warps of one chain).
    // Thread c of the chain owns kPack neighbouring columns of one row: column
    // kPack * (c % (16 / kPack)) of row c / (16 / kPack).
    auto chain = [&](uint32_t k, uint32_t chain_tid, float* chain_lanes, bool scale_finite) {
        const RmsUnit at = rms_locate<G>(p, unit_of(k));
        if (!at.valid) return;                               // uniform per CTA
        constexpr uint32_t kThreadsPerRow = kTile / kPack;
        const bool active = chain_tid < kPairs;
        const uint32_t c = active ? chain_tid : 0;
        const unsigned char* cursor = slot_of(k) + c * (kPack * ELEM);
        float acc0 = 0.0f, acc1 = 0.0f;                      // acc1: the second column (kPack == 2)
        // One load per tile: one element, or two in one word.
        using Raw = typename std::conditional<
                kPack == 1, typename std::conditional<ELEM == 2, uint16_t, float>::type,
                typename std::conditional<ELEM == 2, uint32_t, float2>::type>::type;
        auto first_of = [](Raw raw) {
            if constexpr (kPack == 1 && ELEM == 2) return __uint_as_float(static_cast<uint32_t>(raw) << 16);
            else if constexpr (kPack == 1) return raw;
            else if constexpr (ELEM == 2) return bf16_lo(raw);
            else return raw.x;
        };
        auto second_of = [](Raw raw) {
            if constexpr (kPack == 1) return 0.0f;
            else if constexpr (ELEM == 2) return bf16_hi(raw);
            else return raw.y;
        };
        auto step = [&](Raw raw) {
            if constexpr (kPack == 1) {
                const float x = first_of(raw);
                acc0 = __fadd_rn(acc0, __fmul_rn(x, x));
            } else {
                square_add_pair(acc0, acc1, first_of(raw), second_of(raw));
            }
        };
        // The raw words of kBatch tiles at a time in two register sets: while one set runs
        // through the dependent additions, the loads of the other are in flight (a lane is
        // one addition every four cycles at best; a load from shared memory takes thirty
        // cycles on an idle SM and many times that while the movers stream).
        constexpr uint32_t kBatch = sizeof(Raw) <= 4 ? 32 : 16;
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
            for (uint32_t j = 0; j < kBatch; ++j) step(raw[j]);
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
            step(*reinterpret_cast<const Raw*>(cursor + static_cast<size_t>(tile) * kPieceBytes));
        }
        if (tail_cols != 0) {
            // The ragged last tile: only its logical columns join the sums.
            const Raw raw = *reinterpret_cast<const Raw*>(cursor + static_cast<size_t>(full_tiles) * kPieceBytes);
            const uint32_t column = kPack * (c % kThreadsPerRow);
            const float x0 = first_of(raw), x1 = second_of(raw);
            if (column < tail_cols) acc0 = __fadd_rn(acc0, __fmul_rn(x0, x0));
            if (kPack == 2 && column + 1 < tail_cols) acc1 = __fadd_rn(acc1, __fmul_rn(x1, x1));
        }
        if (active) {
            chain_lanes[kPack * c] = acc0;                   // [row * 16 + column]
            if constexpr (kPack == 2) chain_lanes[kPack * c + 1] = acc1;
        }
        __syncwarp();                                        // a row's threads share a warp
        if (active && (c % kThreadsPerRow) == 0) {
            const uint32_t row = c / kThreadsPerRow;
            const float sum = combine_lanes(chain_lanes + row * kTile);
            inverse[(k % kSlots) * 16 + row] = row_inverse(sum, p.cols, p.eps);
            clean[(k % kSlots) * 16 + row] = row_is_clean(sum, scale_finite) ? 1u : 0u;
        }
    };

    // Fused: sum = x + residual for unit k, rounded to the leaf, kept in the x slot and
    // stored (movers). Each mover keeps its vector position and walks tiles first,
    // + kMoveTilesPerStep, ...
    auto add = [&](uint32_t k) {
        if constexpr (FUSED) {
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
        const RmsUnit at = rms_locate<G>(p, unit_of(k));
        if (!at.valid) return;
        const uint32_t v = mover % kPieceVectors;
        const uint32_t row = v / kVectorsPerRow;
        const uint32_t cv = v % kVectorsPerRow;
        if (row >= min(static_cast<uint32_t>(G), at.rows_in_band - at.row0)) return;
        const uint32_t col_in_tile = cv * kPerVector;
        const uint32_t first_tile = mover / kPieceVectors;
        const float inv = inverse[(k % kSlots) * 16 + row];
        const bool fast = clean[(k % kSlots) * 16 + row] != 0;
        unsigned char* out = rms_unit_base<ELEM>(p, p.out, at) + v * 16
                + static_cast<size_t>(first_tile) * kTileBytes;
        const unsigned char* in = slot_of(k) + static_cast<size_t>(mover) * 16;
        const uint32_t steps = first_tile < full_tiles
                ? (full_tiles - first_tile + kMoveTilesPerStep - 1) / kMoveTilesPerStep : 0;
        constexpr size_t kSlotStep = static_cast<size_t>(kMoveTilesPerStep) * kPieceBytes;
        constexpr size_t kGlobalStep = static_cast<size_t>(kMoveTilesPerStep) * kTileBytes;
        // The walk with the scale in registers: loads of four steps, then their stores.
        auto walk_regs = [&](auto fast_tag) {
            constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
            for (uint32_t first = 0; first < kScaleSteps; first += 4) {
                uint4 xs[4];
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    if (first + j < steps) xs[j] = *reinterpret_cast<const uint4*>(in + (first + j) * kSlotStep);
                }
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    if (first + j < steps) {
                        float w[kPerVector];
                        widen_vector<ELEM>(scale_regs[first + j], w);
                        store_u4_stream(out + (first + j) * kGlobalStep,
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
        // The walk with the scale row widened in shared memory, or read through L1.
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
            const unsigned char* from = in;
            unsigned char* to = out;
            uint32_t step = 0;
            for (; step + 2 <= steps; step += 2) {
                float w0[kPerVector], w1[kPerVector];
                const uint4 x0 = *reinterpret_cast<const uint4*>(from);
                const uint4 x1 = *reinterpret_cast<const uint4*>(from + kSlotStep);
                load_scale(w_cursor, w0);
                load_scale(w_cursor + kScaleStep, w1);
                store_u4_stream(to, normalize_vector<ELEM>(x0, w0, inv, kFast));
                store_u4_stream(to + kGlobalStep, normalize_vector<ELEM>(x1, w1, inv, kFast));
                from += 2 * kSlotStep;
                to += 2 * kGlobalStep;
                w_cursor += 2 * kScaleStep;
            }
            if (step < steps) {
                float w[kPerVector];
                load_scale(w_cursor, w);
                store_u4_stream(to, normalize_vector<ELEM>(*reinterpret_cast<const uint4*>(from), w,
                                                           inv, kFast));
                from += kSlotStep;
                to += kGlobalStep;
                w_cursor += kScaleStep;
            }
            // The ragged last tile, for the thread whose walk reaches it.
            if (tail_cols > col_in_tile && first_tile + steps * kMoveTilesPerStep == full_tiles) {
                float w[kPerVector];
                load_scale(w_cursor, w);
                store_vector_masked<ELEM>(
                        to, normalize_vector<ELEM>(*reinterpret_cast<const uint4*>(from), w, inv, kFast),
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

    // ---- prologue: the barriers, the first copy, then the scale row ----------------
    if (tid == 0) {
        *scale_not_finite = 0;
        *stop = 0;
        for (uint32_t slot = 0; slot < kSlots; ++slot) {
            mbarrier_init(landed_bar + slot, 1);             // the issuing thread (+ the bytes)
            mbarrier_init(added_bar + slot, kMoverWarps);
            mbarrier_init(chained_bar + slot, kChainWarps);
            mbarrier_init(emitted_bar + slot, kMoverWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    for (uint32_t k = 0; k < kCopyAhead; ++k) (void)issue(k);
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

    // ---- the jobs ---------------------------------------------------------------------
    // Who reads what the copy engine wrote waits for that unit's `landed` barrier itself.
    // The jobs have loops of their own, so that neither side's registers count against the
    // other's.
    if (warp < kAllChainWarps) {
        // Chain `mine` takes units mine, mine + kChains, ...
        const uint32_t mine = warp / kChainWarps;
        const uint32_t chain_tid = tid - mine * kChainThreads;
        float* chain_lanes = lanes + mine * G * kTile;
        for (uint32_t k = mine; k < count; k += kChains) {
            if (!await(FUSED ? added_bar : landed_bar, k)) break;
            chain(k, chain_tid, chain_lanes, scale_finite);
            warp_arrives(chained_bar, k);
        }
    } else {
        const bool moves = mover < kMovers;
        if (moves) {
#pragma unroll
            for (uint32_t j = 0; j < kScaleSteps; ++j) scale_regs[j] = make_uint4(0, 0, 0, 0);
            if (shape.scale_in_regs) {
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
        }
        // Step u: unit u + kCopyAhead is issued, unit u added (fused), unit u - kLag emitted.
        for (uint32_t u = 0; u < count + kLag; ++u) {
            if (!issue(u + kCopyAhead)) break;
            if (!moves) continue;
            if constexpr (FUSED) {
                if (u < count) {
                    if (!await(landed_bar, u)) break;
                    add(u);
                    warp_arrives(added_bar, u);
                }
            }
            if (u >= kLag) {
                const uint32_t e = u - kLag;
                if constexpr (!FUSED) {
                    if (!await(landed_bar, e)) break;        // long landed: the chain waited for it
                }
                if (!await(chained_bar, e)) break;
                emit(e);
                warp_arrives(emitted_bar, e);
            }
        }
    }
    // Every job is done, or a wait gave up (it never should). Then copies may still be in
    // flight: give them a bounded time to land before the shared memory goes to another CTA.
    __syncthreads();
    if (*stop != 0 && tid == 0) {
        atomicAdd(&g_rms_copy_timeouts, 1u);
        for (uint32_t slot = 0; slot < kSlots; ++slot) {
            for (uint32_t poll = 0; poll < (1u << 16); ++poll) {
                if (mbarrier_test(landed_bar + slot, 0) || mbarrier_test(landed_bar + slot, 1)) break;
            }
        }
    }
}

using LongKernel = void (*)(const RmsParams, const LongShape, const CUtensorMap, const CUtensorMap);

template <int ELEM, bool FUSED>
static LongKernel pick_long(uint32_t g, uint32_t chains) {
    switch (g) {
        case 16: return rmsnorm_long_kernel<ELEM, 16, FUSED, 1>;
        case 8: return rmsnorm_long_kernel<ELEM, 8, FUSED, 1>;
        case 4: return rmsnorm_long_kernel<ELEM, 4, FUSED, 1>;
        case 2:
            return chains == 3 ? rmsnorm_long_kernel<ELEM, 2, FUSED, 3>
                               : (chains == 2 ? rmsnorm_long_kernel<ELEM, 2, FUSED, 2>
                                              : rmsnorm_long_kernel<ELEM, 2, FUSED, 1>);
        default:
            return chains == 3 ? rmsnorm_long_kernel<ELEM, 1, FUSED, 3>
                               : (chains == 2 ? rmsnorm_long_kernel<ELEM, 1, FUSED, 2>
                                              : rmsnorm_long_kernel<ELEM, 1, FUSED, 1>);
    }
}

int prepare_rmsnorm_long_kernels() {
    for (uint32_t g = 1; g <= kTile; g *= 2) {
        for (uint32_t chains = 1; chains <= kMaxChains; ++chains) {
            const LongKernel kernels[4] = {pick_long<2, false>(g, chains), pick_long<2, true>(g, chains),
                                           pick_long<4, false>(g, chains), pick_long<4, true>(g, chains)};
            for (const LongKernel kernel : kernels) {
                const int status = allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
                if (status != IOMB_OK) return status;
            }
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
    // whole boxes. Largest group of rows of which the slots (and the rest) fit one SM.
    const uint32_t boxes = (base.tile_cols + kMaxBoxTiles - 1) / kMaxBoxTiles;
    // (a multiple of four tiles, so that every box starts on a 128-byte boundary of its slot)
    const uint32_t box_tiles = ((base.tile_cols + boxes - 1) / boxes + 3) / 4 * 4;
    const uint64_t slot_row_bytes = static_cast<uint64_t>(boxes) * box_tiles * kTile * elem;
    auto slot_bytes = [&](uint32_t rows, uint32_t chains) {
        return long_slots(fused, chains) * rows * slot_row_bytes;
    };
    auto fits = [&](uint32_t rows, uint32_t chains) {
        return slot_bytes(rows, chains) + long_fixed_bytes(rows, fused, chains) <= kSharedCap;
    };
    if (!fits(1, 1)) return IOMB_OK;                       // not served here
    // Few rows (decode steps): smaller groups spread the bands over more SMs.
    const uint64_t sms = static_cast<uint64_t>(sm_count() > 0 ? sm_count() : 148);
    uint32_t largest = kTile;
    while (largest > 1 && bands * (kTile / largest) < sms) largest /= 2;
    // Rows chaining at once on an SM are g * chains: about four keep up with HBM (measured:
    // g 4 with one chain unfused, g 2 with two chains fused; g 2 with one chain runs at half
    // the rate). Among the shapes that fit, take the one with the most, then the tallest
    // group, then the fewest chains.
    uint32_t g = 0, chains = 1, best = 0;
    for (uint32_t rows = largest; rows >= 1; rows /= 2) {
        for (uint32_t c = 1; c <= long_most_chains(rows, fused); ++c) {
            if (!fits(rows, c)) continue;
            const uint32_t chaining = rows * c < 4 ? rows * c : 4;
            if (chaining > best) {
                best = chaining;
                g = rows;
                chains = c;
            }
        }
    }
    if (g == 0) return IOMB_OK;
    const uint64_t scale_bytes = row_bytes / elem * 4;     // row 0 of every scale tile as FP32
    LongShape shape{};
    shape.boxes = boxes;
    shape.box_tiles = box_tiles;
    const uint64_t walk_tiles = long_move_tiles_per_step(elem, g, fused, chains);
    shape.scale_in_regs = (base.tile_cols + walk_tiles - 1) / walk_tiles <= long_scale_steps(fused) ? 1u : 0u;
    shape.scale_in_smem = !shape.scale_in_regs
                    && slot_bytes(g, chains) + scale_bytes + long_fixed_bytes(g, fused, chains) <= kSharedCap
            ? 1u : 0u;
    const uint64_t smem_bytes = slot_bytes(g, chains) + (shape.scale_in_smem ? scale_bytes : 0)
            + long_fixed_bytes(g, fused, chains);

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
            ? (fused ? pick_long<2, true>(g, chains) : pick_long<2, false>(g, chains))
            : (fused ? pick_long<4, true>(g, chains) : pick_long<4, false>(g, chains));
    const int prepared = allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
    if (prepared != IOMB_OK) return prepared;
    // The CTAs of a launch start on neighbouring units (the groups of one band, then the
    // next band) and nothing keeps them in step afterwards. Once they have drifted apart,
    // the 64- or 128-byte pieces of one tile are fetched at different times and DRAM opens a
    // row for each piece: measured on [262144, 8192] BF16, one launch ran at 0.55 of the
    // rate of the same rows in launches of 32768. So a launch covers a bounded number of
    // units per CTA (equal launches: a short last one would run at a lower rate); the
    // launches of one call follow one another on the stream.
    const uint64_t all_units = p.units;
    const uint64_t per_cta = (all_units + sms - 1) / sms;
    const uint64_t parts = (per_cta + kUnitsPerCtaAndLaunch - 1) / kUnitsPerCtaAndLaunch;
    const uint64_t per_launch = sms * ((per_cta + parts - 1) / parts);     // equal launches
    uint32_t launches = 0;
    for (uint64_t first = 0; first < all_units; first += per_launch, ++launches) {
        p.first_unit = first;
        p.units = all_units - first < per_launch ? all_units - first : per_launch;
        const uint64_t grid = p.units < sms ? p.units : sms;
        kernel<<<static_cast<unsigned>(grid), kLongThreads, smem_bytes, stream>>>(p, shape, x_map, r_map);
    }
    const uint64_t grid = all_units < sms ? all_units : sms;
    *launched = true;
    char text[160];
    snprintf(text, sizeof text,
             "rmsnorm_long_kernel<elem %u, rows %u, %s> %u chain(s), %u slots, scale %s, %u CTAs x %d, %u launch(es)",
             elem, g, fused ? "fused" : "unfused", chains, long_slots(fused, chains),
             shape.scale_in_regs ? "in registers" : shape.scale_in_smem ? "in shared memory" : "through L1",
             static_cast<unsigned>(grid), kLongThreads, launches);
    note_launch(text);
    return check_launch("rmsnorm launch");
}

}  // namespace iomb

extern "C" int iomb_rmsnorm_copy_timeouts(unsigned int* count) {
    if (count == nullptr) return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "iomb_rmsnorm_copy_timeouts: null result");
    if (cudaMemcpyFromSymbol(count, iomb::g_rms_copy_timeouts, sizeof(unsigned int)) != cudaSuccess) {
        return iomb::fail(IOMB_ERR_DEVICE, "iomb_rmsnorm_copy_timeouts: reading the counter failed");
    }
    return IOMB_OK;
}
