// Split-half rotary position embedding on tiled storage.
//
// Replaces GpuQueue::rope_impl + the word-owner kernel of the reference
// (src/shared/standard_tiled_rope.inl:83-624). Semantics are those of the CPU
// backend (src/cpu/queue.cpp:1338-1592): x is [..., H, R, W]; row r of every
// plane sits at position a + r; columns c and c + W/2 form a pair that is rotated
// by angle(position, c) with four separately rounded FP32 products, one
// subtraction and one addition, and one RNE encode per result; a row at position 0
// is copied raw.
//
// The angles do not depend on the data, and the reference fixes them as the C
// library's powf / sinf / cosf of the host (src/cpu/queue.cpp:1356-1367), so they
// are not recomputed on the device: iomb_rope_angles fills a (cos, sin) table on
// the host with exactly those expressions, the caller keeps it in device memory
// (a rotary cache, as serving engines keep one) and iomb_rope reads the rows it
// needs. Results are then bit-identical to the reference CPU backend on the same
// host. A warp owns one tile of the first half and its partner tile of the second
// half (two contiguous 512/1024-byte pieces read, two written) for a group of
// planes that share the tile's angles.
#include "host.hpp"

#include <math.h>

namespace iomb {

constexpr int kRopeThreads = 256;

struct RopeParams {
    Operand x;
    Operand out;
    Leading leading;
    uint32_t rows;
    uint32_t cols;
    uint32_t half;
    uint32_t tile_rows;
    uint32_t tile_cols;
    uint32_t half_tiles;       // tiles of the first half (fast path: half % 16 == 0)
    uint64_t first_position;   // a
    uint64_t items;            // fast: plane groups * tile_rows * half_tiles; slow: planes * rows * half
    const float2* angles;      // [rows][half] (cos, sin), row 0 = position a
};

__device__ __forceinline__ void rotate(float first, float second, float2 angle, float& first_out,
                                       float& second_out) {
    first_out = __fsub_rn(__fmul_rn(first, angle.x), __fmul_rn(second, angle.y));
    second_out = __fadd_rn(__fmul_rn(second, angle.x), __fmul_rn(first, angle.y));
}

// Fast path: W/2 is a multiple of 16, so a pair's two columns sit at the same
// place of two different tiles. One warp per (band, tile of the first half, group
// of kRopePlanes planes): the angles of the tile are loaded once and kept in
// registers while the warp walks the group's planes (heads and sequences share them).
constexpr uint32_t kRopePlanes = 16;
constexpr uint32_t kRopeBatch = 2;

template <int ELEM>
__global__ void __launch_bounds__(kRopeThreads, 4)
rope_tile_kernel(const RopeParams p) {
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kTileVectors = kTileBytes / 16;
    constexpr uint32_t kPerVector = 16 / ELEM;
    constexpr uint32_t kVectorsPerRow = kTile / kPerVector;
    constexpr int kWarps = kRopeThreads / 32;
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kWarps;
    for (uint64_t item = warp; item < p.items; item += warps) {
        // item = ((group * tile_rows) + tr) * half_tiles + tc: neighbouring warps share a band
        const uint32_t tc = static_cast<uint32_t>(item % p.half_tiles);
        const uint64_t rest = item / p.half_tiles;
        const uint32_t tr = static_cast<uint32_t>(rest % p.tile_rows);
        const uint64_t group = rest / p.tile_rows;
        const uint64_t first_tile = static_cast<uint64_t>(tr) * p.tile_cols + tc;
        const uint32_t rows_left = p.rows - tr * kTile;
        const uint64_t first_plane = group * kRopePlanes;
        const uint32_t planes_here = static_cast<uint32_t>(
                min(static_cast<uint64_t>(kRopePlanes), p.leading.planes - first_plane));
        for (uint32_t k = lane; k < kTileVectors; k += 32) {
            const uint32_t row_in_tile = k / kVectorsPerRow;
            if (row_in_tile >= rows_left) continue;
            const uint32_t column = tc * kTile + (k % kVectorsPerRow) * kPerVector;
            const uint32_t row = tr * kTile + row_in_tile;
            const bool raw_copy = p.first_position + row == 0;     // position 0
            float2 angle[kPerVector];
            if (!raw_copy) {
                const float4* source = reinterpret_cast<const float4*>(
                        p.angles + static_cast<size_t>(row) * p.half + column);
#pragma unroll
                for (uint32_t w = 0; w < kPerVector / 2; ++w) {
                    const float4 two = __ldg(source + w);          // (cos, sin) of two columns
                    angle[2 * w] = make_float2(two.x, two.y);
                    angle[2 * w + 1] = make_float2(two.z, two.w);
                }
            }
            const size_t partner = static_cast<size_t>(p.half_tiles) * kTileBytes;
            // kRopeBatch planes' vectors are in flight before the first is rotated.
            for (uint32_t q0 = 0; q0 < planes_here; q0 += kRopeBatch) {
                uint4 a[kRopeBatch], b[kRopeBatch];
                unsigned char* target[kRopeBatch];
#pragma unroll
                for (uint32_t u = 0; u < kRopeBatch; ++u) {
                    if (q0 + u >= planes_here) continue;
                    const uint64_t x_plane = operand_plane(p.x, p.leading, first_plane + q0 + u);
                    const uint64_t out_plane = operand_plane(p.out, p.leading, first_plane + q0 + u);
                    const unsigned char* x_first = p.x.base
                            + (x_plane * p.tile_rows * p.tile_cols + first_tile) * kTileBytes + k * 16;
                    target[u] = p.out.base
                            + (out_plane * p.tile_rows * p.tile_cols + first_tile) * kTileBytes + k * 16;
                    a[u] = load_u4_stream(x_first);
                    b[u] = load_u4_stream(x_first + partner);
                }
#pragma unroll
                for (uint32_t u = 0; u < kRopeBatch; ++u) {
                    if (q0 + u >= planes_here) continue;
                    uint4 ra = a[u], rb = b[u];
                    if (!raw_copy) {
                        const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
                        const uint32_t bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
                        uint32_t ow[4], pw[4];
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            if constexpr (ELEM == 2) {
                                float f0, s0, f1, s1;
                                rotate(bf16_lo(aw[w]), bf16_lo(bw[w]), angle[2 * w], f0, s0);
                                rotate(bf16_hi(aw[w]), bf16_hi(bw[w]), angle[2 * w + 1], f1, s1);
                                ow[w] = pack_bf16x2_canonical(f0, f1);
                                pw[w] = pack_bf16x2_canonical(s0, s1);
                            } else {
                                float f, s2;
                                rotate(__uint_as_float(aw[w]), __uint_as_float(bw[w]), angle[w], f, s2);
                                ow[w] = f32_canonical_bits(f);
                                pw[w] = f32_canonical_bits(s2);
                            }
                        }
                        ra = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                        rb = make_uint4(pw[0], pw[1], pw[2], pw[3]);
                    }
                    store_u4_stream(target[u], ra);
                    store_u4_stream(target[u] + partner, rb);
                }
            }
        }
    }
}

// Any even width: one thread per pair.
template <int ELEM>
__global__ void __launch_bounds__(kRopeThreads)
rope_pair_kernel(const RopeParams p) {
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    const uint64_t thread = static_cast<uint64_t>(blockIdx.x) * kRopeThreads + threadIdx.x;
    const uint64_t threads = static_cast<uint64_t>(gridDim.x) * kRopeThreads;
    for (uint64_t item = thread; item < p.items; item += threads) {
        const uint32_t column = static_cast<uint32_t>(item % p.half);
        const uint64_t rest = item / p.half;
        const uint32_t row = static_cast<uint32_t>(rest % p.rows);
        const uint64_t index = rest / p.rows;
        auto slot = [&](const Operand& operand, uint32_t c) {
            const uint64_t plane = operand_plane(operand, p.leading, index);
            const uint64_t tile = static_cast<uint64_t>(row / kTile) * p.tile_cols + c / kTile;
            return operand.base + (plane * p.tile_rows * p.tile_cols + tile) * kTileBytes
                    + ((row % kTile) * kTile + c % kTile) * ELEM;
        };
        const unsigned char* xa = slot(p.x, column);
        const unsigned char* xb = slot(p.x, column + p.half);
        unsigned char* oa = slot(p.out, column);
        unsigned char* ob = slot(p.out, column + p.half);
        if constexpr (ELEM == 2) {
            const uint16_t a = *reinterpret_cast<const uint16_t*>(xa);
            const uint16_t b = *reinterpret_cast<const uint16_t*>(xb);
            uint16_t ra = a, rb = b;
            if (p.first_position + row != 0) {
                float f, s;
                rotate(__uint_as_float(static_cast<uint32_t>(a) << 16),
                       __uint_as_float(static_cast<uint32_t>(b) << 16),
                       __ldg(p.angles + static_cast<size_t>(row) * p.half + column), f, s);
                const uint32_t packed = pack_bf16x2_canonical(f, s);
                ra = static_cast<uint16_t>(packed & 0xFFFFu);
                rb = static_cast<uint16_t>(packed >> 16);
            }
            *reinterpret_cast<uint16_t*>(oa) = ra;
            *reinterpret_cast<uint16_t*>(ob) = rb;
        } else {
            const uint32_t a = *reinterpret_cast<const uint32_t*>(xa);
            const uint32_t b = *reinterpret_cast<const uint32_t*>(xb);
            uint32_t ra = a, rb = b;
            if (p.first_position + row != 0) {
                float f, s;
                rotate(__uint_as_float(a), __uint_as_float(b),
                       __ldg(p.angles + static_cast<size_t>(row) * p.half + column), f, s);
                ra = f32_canonical_bits(f);
                rb = f32_canonical_bits(s);
            }
            *reinterpret_cast<uint32_t*>(oa) = ra;
            *reinterpret_cast<uint32_t*>(ob) = rb;
        }
    }
}

}  // namespace iomb

// rope_angle of the reference CPU backend (src/cpu/queue.cpp:1356-1367) on the FP32
// carrier, for positions first_position .. first_position + rows - 1 and the W/2
// columns of the first half: cos_sin[(r * W/2 + c) * 2 + {0, 1}] = {cos, sin}.
// Host code: the C library's powf / sinf / cosf are part of the definition.
extern "C" int iomb_rope_angles(float* cos_sin, uint64_t first_position, uint64_t rows,
                                uint64_t width, double theta) {
    if (cos_sin == nullptr || width == 0 || width % 2 != 0) {
        return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "rope_angles: width must be positive and even");
    }
    if (!(theta >= 1.0) || theta > 3.4028234663852886e38) {
        return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "rope theta must be finite in [1,float_max]");
    }
    const float narrowed = static_cast<float>(theta);
    const uint64_t half = width / 2;
    for (uint64_t r = 0; r < rows; ++r) {
        const float position = static_cast<float>(first_position + r);
        for (uint64_t c = 0; c < half; ++c) {
            const float exponent = static_cast<float>(
                    (-2.0 * static_cast<double>(c)) / static_cast<double>(width));
            const float frequency = powf(narrowed, exponent);
            const float angle = position * frequency;
            cos_sin[(r * half + c) * 2] = cosf(angle);
            cos_sin[(r * half + c) * 2 + 1] = sinf(angle);
        }
    }
    return IOMB_OK;
}

extern "C" int iomb_rope(const iomb_view* x, const iomb_view* out, uint64_t a,
                         const float* cos_sin, void* stream) {
    using namespace iomb;
    ViewFacts fx{}, fo{};
    int status = check_view(x, "rope x", &fx);
    if (status == IOMB_OK) status = check_view(out, "rope out", &fo);
    if (status != IOMB_OK) return status;
    // Admission order of validate_rope (src/device_ops_neural.cpp:241-360).
    if (x->rank < 3 || out->rank != x->rank) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rope requires rank three through eight");
    }
    for (uint32_t i = 0; i < x->rank; ++i) {
        if (x->dims[i] != out->dims[i]) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "rope input and output shapes must match");
        }
    }
    if (fx.cols % 2 != 0) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rope final width must be positive and even");
    }
    // The last position, a + R - 1, must stay below 2^24 (exact in binary32).
    constexpr uint64_t kMaxPosition = (1ull << 24) - 1;
    if (a > kMaxPosition || fx.rows - 1 > kMaxPosition - a) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rope position exceeds the binary32 bound");
    }
    if (out->base == x->base || storage_overlaps(*out, fo, *x, fx)) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rope output aliases or overlaps the input");
    }
    if (x->dtype != out->dtype) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rope input and output specifications must match");
    }
    if (x->dtype != IOMB_BF16 && x->dtype != IOMB_F32) {
        return fail(IOMB_ERR_UNSUPPORTED, "rope: leaf is not BF16 or F32");
    }
    if (cos_sin == nullptr) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "rope: the angle table is required");
    }
    if (fx.rows > 0xFFFFFFFFull || fx.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "rope: matrix extent exceeds the kernel limit");
    }
    RopeParams p{};
    uint64_t strides[2][kMaxLead] = {};
    for (uint32_t axis = 0; axis < fx.leading; ++axis) {
        strides[0][axis] = x->plane_strides[axis];
        strides[1][axis] = out->plane_strides[axis];
    }
    collapse_leading(fx.leading, x->dims, strides, 2, &p.leading);
    p.x = make_operand(*x, fx, strides[0], p.leading, false, false);
    p.out = make_operand(*out, fo, strides[1], p.leading, false, false);
    p.rows = static_cast<uint32_t>(fx.rows);
    p.cols = static_cast<uint32_t>(fx.cols);
    p.half = p.cols / 2;
    p.tile_rows = static_cast<uint32_t>(fx.tile_rows);
    p.tile_cols = static_cast<uint32_t>(fx.tile_cols);
    p.first_position = a;
    p.angles = reinterpret_cast<const float2*>(cos_sin);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (p.half % kTile == 0) {
        p.half_tiles = p.half / kTile;
        p.items = ((p.leading.planes + kRopePlanes - 1) / kRopePlanes) * fx.tile_rows * p.half_tiles;
        const unsigned grid = grid_one_shot((p.items + kRopeThreads / 32 - 1) / (kRopeThreads / 32));
        if (x->dtype == IOMB_BF16) rope_tile_kernel<2><<<grid, kRopeThreads, 0, s>>>(p);
        else rope_tile_kernel<4><<<grid, kRopeThreads, 0, s>>>(p);
    } else {
        p.items = p.leading.planes * fx.rows * p.half;
        const unsigned grid = grid_one_shot((p.items + kRopeThreads - 1) / kRopeThreads);
        if (x->dtype == IOMB_BF16) rope_pair_kernel<2><<<grid, kRopeThreads, 0, s>>>(p);
        else rope_pair_kernel<4><<<grid, kRopeThreads, 0, s>>>(p);
    }
    return check_launch("rope launch");
}
