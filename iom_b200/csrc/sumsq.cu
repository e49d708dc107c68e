// Whole-view FP32 sum of squares with an order that does not depend on the
// launch geometry. No counterpart in the reference.
//
// The view's tiles are cut into kSlots contiguous runs, one per logical
// accumulator. A CTA serves one slot at a time: thread t of the CTA squares and adds its share of
// every tile of the slot in tile order (masked to the logical extents), the 256
// thread sums are folded by a fixed shared-memory tree into partial[slot], and
// the CTA that finishes last folds the kSlots partials the same way. Which CTA
// ran which slot, and how many CTAs there were, never changes a bit of the
// result.
#include "host.hpp"

namespace iomb {

constexpr int kSumThreads = 256;
constexpr uint32_t kSlots = 2048;
// Scratch: kSlots partial sums followed by one completion counter.
constexpr uint64_t kScratchBytes = kSlots * sizeof(float) + 32;

struct SumsqParams {
    Operand x;
    Leading leading;
    uint32_t rows;
    uint32_t cols;
    uint32_t tile_rows;
    uint32_t tile_cols;
    uint32_t elem;
    uint64_t tiles;      // planes * tile_rows * tile_cols
    float* partial;
    uint32_t* counter;
    float* result;
};

__device__ __forceinline__ float fold_block(float value, float* shared) {
    shared[threadIdx.x] = value;
    __syncthreads();
    for (int step = kSumThreads / 2; step > 0; step >>= 1) {
        if (static_cast<int>(threadIdx.x) < step) {
            shared[threadIdx.x] = __fadd_rn(shared[threadIdx.x], shared[threadIdx.x + step]);
        }
        __syncthreads();
    }
    const float total = shared[0];
    __syncthreads();
    return total;
}

// 256 threads cover one tile: 16-bit leaves as 32 vectors of 8 elements (the
// first 32 threads), 32-bit leaves as 64 vectors of 4 elements. To keep every
// thread busy a CTA walks 8 (16-bit) or 4 (32-bit) consecutive tiles of its
// slot at once.
template <int ELEM, bool DENSE>
__global__ void __launch_bounds__(kSumThreads)
sumsq_kernel(const SumsqParams p) {
    __shared__ float shared[kSumThreads];
    __shared__ uint32_t last;
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kTileVectors = kTileBytes / 16;
    constexpr uint32_t kTilesPerStep = kSumThreads / kTileVectors;
    constexpr uint32_t kPerVector = 16 / ELEM;
    const uint32_t sub = threadIdx.x / kTileVectors;       // which tile of the step
    const uint32_t vector = threadIdx.x % kTileVectors;
    const uint32_t slot_in_tile = vector * kPerVector;
    const uint32_t row = slot_in_tile / kTile, col = slot_in_tile % kTile;
    const uint64_t groups = (p.tiles + kTilesPerStep - 1) / kTilesPerStep;
    const uint64_t per_slot = (groups + kSlots - 1) / kSlots;   // contiguous run per slot
    for (uint32_t slot = blockIdx.x; slot < kSlots; slot += gridDim.x) {
        float acc = 0.0f;
        // Four tiles of the slot are fetched before any is added; the adds keep
        // tile order, so batching does not change the result.
        constexpr uint32_t kBatch = 4;
        const uint64_t begin = slot * per_slot;
        const uint64_t end = min(begin + per_slot, groups);
        for (uint64_t group0 = begin; group0 < end; group0 += kBatch) {
            uint4 v[kBatch];
            uint32_t valid[kBatch];
#pragma unroll
            for (uint32_t b = 0; b < kBatch; ++b) {
                valid[b] = 0;
                const uint64_t group = group0 + b;
                const uint64_t tile = group * kTilesPerStep + sub;
                if (group >= end || tile >= p.tiles) continue;
                if constexpr (DENSE) {
                    // Tile-multiple extents and dense planes: tiles are consecutive.
                    valid[b] = kPerVector;
                    v[b] = load_u4_stream(p.x.base + tile * kTileBytes + vector * 16);
                } else {
                    const uint32_t tc = static_cast<uint32_t>(tile % p.tile_cols);
                    const uint64_t band = tile / p.tile_cols;
                    const uint32_t tr = static_cast<uint32_t>(band % p.tile_rows);
                    const uint64_t index = band / p.tile_rows;
                    const uint32_t rows_left = p.rows - tr * kTile;
                    const uint32_t cols_left = p.cols - tc * kTile;
                    if (row >= rows_left || col >= cols_left) continue;
                    valid[b] = min(kPerVector, cols_left - col);
                    v[b] = load_u4_stream(
                            p.x.base
                            + (operand_plane(p.x, p.leading, index) * p.tile_rows * p.tile_cols
                               + static_cast<uint64_t>(tr) * p.tile_cols + tc) * kTileBytes
                            + vector * 16);
                }
            }
#pragma unroll
            for (uint32_t b = 0; b < kBatch; ++b) {
                if (valid[b] == 0) continue;
                float e[8];
                if constexpr (ELEM == 2) {
                    e[0] = bf16_lo(v[b].x); e[1] = bf16_hi(v[b].x);
                    e[2] = bf16_lo(v[b].y); e[3] = bf16_hi(v[b].y);
                    e[4] = bf16_lo(v[b].z); e[5] = bf16_hi(v[b].z);
                    e[6] = bf16_lo(v[b].w); e[7] = bf16_hi(v[b].w);
                } else {
                    e[0] = __uint_as_float(v[b].x); e[1] = __uint_as_float(v[b].y);
                    e[2] = __uint_as_float(v[b].z); e[3] = __uint_as_float(v[b].w);
                }
#pragma unroll
                for (uint32_t k = 0; k < kPerVector; ++k) {
                    if (k < valid[b]) acc = __fadd_rn(acc, __fmul_rn(e[k], e[k]));
                }
            }
        }
        const float total = fold_block(acc, shared);
        if (threadIdx.x == 0) p.partial[slot] = total;
    }
    // The CTA that finishes last folds the partials in slot order.
    __threadfence();
    if (threadIdx.x == 0) {
        last = atomicAdd(p.counter, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (last) {
        __threadfence();
        float acc = 0.0f;
        for (uint32_t slot = threadIdx.x; slot < kSlots; slot += kSumThreads) {
            acc = __fadd_rn(acc, __ldcg(p.partial + slot));
        }
        const float total = fold_block(acc, shared);
        if (threadIdx.x == 0) {
            *p.result = total;
            *p.counter = 0;
        }
    }
}

}  // namespace iomb

extern "C" uint64_t iomb_sumsq_scratch_bytes(void) { return iomb::kScratchBytes; }

extern "C" int iomb_sumsq(const iomb_view* x, void* scratch, float* result, void* stream) {
    using namespace iomb;
    ViewFacts f{};
    const int rc = check_view(x, "sumsq x", &f);
    if (rc != IOMB_OK) return rc;
    if (scratch == nullptr || result == nullptr) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "sumsq: scratch and result are required");
    }
    if (reinterpret_cast<uintptr_t>(scratch) % 16 != 0) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "sumsq: scratch must be 16-byte aligned");
    }
    if (x->dtype != IOMB_BF16 && x->dtype != IOMB_F32) {
        return fail(IOMB_ERR_UNSUPPORTED, "sumsq: leaf is not BF16 or F32");
    }
    if (f.rows > 0xFFFFFFFFull || f.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "sumsq: matrix extent exceeds the kernel limit");
    }
    SumsqParams p{};
    uint64_t strides[1][kMaxLead] = {};
    for (uint32_t axis = 0; axis < f.leading; ++axis) strides[0][axis] = x->plane_strides[axis];
    collapse_leading(f.leading, x->dims, strides, 1, &p.leading);
    p.x = make_operand(*x, f, strides[0], p.leading, false, false);
    p.rows = static_cast<uint32_t>(f.rows);
    p.cols = static_cast<uint32_t>(f.cols);
    p.tile_rows = static_cast<uint32_t>(f.tile_rows);
    p.tile_cols = static_cast<uint32_t>(f.tile_cols);
    p.elem = f.bytes;
    p.tiles = p.leading.planes * f.tile_rows * f.tile_cols;
    p.partial = static_cast<float*>(scratch);
    p.counter = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(scratch)
                                            + kSlots * sizeof(float));
    p.result = result;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The completion counter must start at zero whatever the scratch held.
    if (cudaMemsetAsync(p.counter, 0, sizeof(uint32_t), s) != cudaSuccess) {
        return check_launch("sumsq counter reset");
    }
    const unsigned grid = kSlots;
    const bool dense = p.leading.contiguous && f.rows % kTile == 0 && f.cols % kTile == 0;
    if (dense) p.x.base += x->plane_offset * f.plane_bytes;
    if (f.bytes == 2) {
        if (dense) sumsq_kernel<2, true><<<grid, kSumThreads, 0, s>>>(p);
        else sumsq_kernel<2, false><<<grid, kSumThreads, 0, s>>>(p);
    } else {
        if (dense) sumsq_kernel<4, true><<<grid, kSumThreads, 0, s>>>(p);
        else sumsq_kernel<4, false><<<grid, kSumThreads, 0, s>>>(p);
    }
    return check_launch("sumsq launch");
}

// ---- sum of squares without caller scratch -----------------------------------
//
// Some hosts of this library have no scratch to hand over and are not allowed
// to create any: IOM's backend contract gives operations such as rmsnorm a
// workspace requirement of {0, 1} (the caller passes none) and forbids every
// native allocation once the device is set up, and a hook that runs while a
// serving loop has frozen its memory pools is in the same position. For them the
// partial sums live in a fixed array that is part of the library image. Every
// GPU that loads the library carries the array until the process exits.
namespace iomb {

constexpr uint64_t kStaticScratchBytes = 16 * 1024;                 // capacity of the array
constexpr uint64_t kStaticMaxElements = IOMB_SUMSQ_STATIC_MAX_ELEMENTS;   // largest view served

static __device__ __align__(256) unsigned char g_sumsq_static_scratch[kStaticScratchBytes];

// Device address of the array, looked up once per device ordinal. The array's
// name is only a host-side handle; kernels must be given the looked-up address.
static void* g_static_scratch_address[64];
static int static_scratch(void** address) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        cudaGetLastError();
        return fail(IOMB_ERR_DEVICE, "sumsq_static: no current CUDA device");
    }
    void* known = __atomic_load_n(&g_static_scratch_address[device], __ATOMIC_ACQUIRE);
    if (known == nullptr) {
        void* looked_up = nullptr;
        const cudaError_t status = cudaGetSymbolAddress(&looked_up, g_sumsq_static_scratch);
        if (status != cudaSuccess || looked_up == nullptr) {
            cudaGetLastError();
            return fail(IOMB_ERR_DEVICE, "sumsq_static: the scratch array's device address is unavailable");
        }
        __atomic_store_n(&g_static_scratch_address[device], looked_up, __ATOMIC_RELEASE);
        known = looked_up;
    }
    *address = known;
    return IOMB_OK;
}

}  // namespace iomb

extern "C" int iomb_sumsq_static(const iomb_view* x, float* result, void* stream) {
    using namespace iomb;
    static_assert(kScratchBytes <= kStaticScratchBytes, "the static array must hold the partials");
    ViewFacts f{};
    const int rc = check_view(x, "sumsq_static x", &f);
    if (rc != IOMB_OK) return rc;
    // planes * rows * cols cannot overflow here: check_view bounded the storage.
    const long double elements =
            static_cast<long double>(f.planes) * static_cast<long double>(f.rows)
            * static_cast<long double>(f.cols);
    if (elements > static_cast<long double>(kStaticMaxElements)) {
        return fail(IOMB_ERR_INVALID_ARGUMENT,
                    "sumsq_static: the view has more than 2^32 elements; use iomb_sumsq with "
                    "caller scratch");
    }
    if (iomb_sumsq_scratch_bytes() > kStaticScratchBytes) {
        return fail(IOMB_ERR_INTERNAL, "sumsq_static: partials exceed the static array");
    }
    void* scratch = nullptr;
    const int lookup = static_scratch(&scratch);
    if (lookup != IOMB_OK) return lookup;
    // The shared launch path resets the completion counter in stream order and
    // every partial is overwritten before it is read, so what an earlier call
    // left in the array never reaches the result.
    return iomb_sumsq(x, scratch, result, stream);
}
