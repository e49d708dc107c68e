// Bit-exact view copy, BF16<->F32 conversion and host-layout scatter/gather on
// tiled storage.
//
// Replaces the word-owner read-modify-write kernels of the reference
// (grid_stride_copy_kernel, src/shared/standard_tiled_copy_metadata.inl:177-282;
// scatter_plane_kernel / gather_plane_kernel with one launch per plane,
// src/shared/standard_tiled_copy.inl:286-441). Here a warp owns whole tiles and
// moves them as 16-byte vectors; logical bounds mask the stores, so padding and
// unselected planes are never written; all planes of a view go in one launch.
#include "host.hpp"

namespace iomb {

constexpr int kCopyThreads = 256;
constexpr int kCopyWarps = kCopyThreads / 32;
constexpr int kCopyUnroll = 4;

enum class Move : int { Copy = 0, Bf16ToF32 = 1, F32ToBf16 = 2 };

// ---- element conversion ---------------------------------------------------

// BF16 -> F32: exact widening; a NaN becomes the positive quiet NaN
// (decode of src/shared/scalar_binary_codec.hpp:45-56 drops sign and payload).
__device__ __forceinline__ uint32_t widen_bf16(uint32_t half) {
    const uint32_t bits = half << 16;
    return (bits & 0x7FFFFFFFu) > 0x7F800000u ? 0x7FC00000u : bits;
}

__device__ __forceinline__ void widen_vector(uint4 in, uint4* lo, uint4* hi) {
    *lo = make_uint4(widen_bf16(in.x & 0xFFFFu), widen_bf16(in.x >> 16),
                     widen_bf16(in.y & 0xFFFFu), widen_bf16(in.y >> 16));
    *hi = make_uint4(widen_bf16(in.z & 0xFFFFu), widen_bf16(in.z >> 16),
                     widen_bf16(in.w & 0xFFFFu), widen_bf16(in.w >> 16));
}

__device__ __forceinline__ uint4 narrow_vectors(uint4 lo, uint4 hi) {
    return make_uint4(
            pack_bf16x2_canonical(__uint_as_float(lo.x), __uint_as_float(lo.y)),
            pack_bf16x2_canonical(__uint_as_float(lo.z), __uint_as_float(lo.w)),
            pack_bf16x2_canonical(__uint_as_float(hi.x), __uint_as_float(hi.y)),
            pack_bf16x2_canonical(__uint_as_float(hi.z), __uint_as_float(hi.w)));
}

// ---- linear streams ---------------------------------------------------------

// One contiguous chunk of kCopyThreads * kCopyUnroll vectors per CTA.
__global__ void __launch_bounds__(kCopyThreads)
copy_linear_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, uint64_t vectors) {
    constexpr uint64_t kChunk = static_cast<uint64_t>(kCopyThreads) * kCopyUnroll;
    const uint64_t chunks = (vectors + kChunk - 1) / kChunk;
    for (uint64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
        const uint64_t base = chunk * kChunk + threadIdx.x;
        if (base + kCopyThreads * (kCopyUnroll - 1) < vectors) {
            // A whole chunk: pairs of neighbouring vectors as 256-bit accesses.
            uint4 v[kCopyUnroll];
            const uint64_t pair = (chunk * kChunk) / 2 + threadIdx.x;
#pragma unroll
            for (int u = 0; u < kCopyUnroll / 2; ++u) {
                load_u8_stream(src + 2 * (pair + u * kCopyThreads), &v[2 * u], &v[2 * u + 1]);
            }
#pragma unroll
            for (int u = 0; u < kCopyUnroll / 2; ++u) {
                store_u8_stream(dst + 2 * (pair + u * kCopyThreads), v[2 * u], v[2 * u + 1]);
            }
        } else {
            for (int u = 0; u < kCopyUnroll; ++u) {
                const uint64_t index = base + u * kCopyThreads;
                if (index < vectors) store_u4_stream(dst + index, load_u4_stream(src + index));
            }
        }
    }
}

// `groups` counts runs of 8 elements: 16 bytes of BF16, 32 bytes of F32.
template <Move M>
__global__ void __launch_bounds__(kCopyThreads)
cast_linear_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, uint64_t groups) {
    constexpr int kBatch = 4;
    constexpr uint64_t kChunk = static_cast<uint64_t>(kCopyThreads) * kBatch;
    const uint64_t chunks = (groups + kChunk - 1) / kChunk;
    for (uint64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
        const uint64_t base = chunk * kChunk + threadIdx.x;
        const bool whole = base + kCopyThreads * (kBatch - 1) < groups;
        if constexpr (M == Move::Bf16ToF32) {
            uint4 in[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint64_t index = base + u * kCopyThreads;
                if (whole || index < groups) in[u] = load_u4_stream(src + index);
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint64_t index = base + u * kCopyThreads;
                if (whole || index < groups) {
                    uint4 lo, hi;
                    widen_vector(in[u], &lo, &hi);
                    store_u8_stream(dst + 2 * index, lo, hi);
                }
            }
        } else {
            uint4 lo[kBatch], hi[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint64_t index = base + u * kCopyThreads;
                if (whole || index < groups) {
                    load_u8_stream(src + 2 * index, &lo[u], &hi[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint64_t index = base + u * kCopyThreads;
                if (whole || index < groups) {
                    store_u4_stream(dst + index, narrow_vectors(lo[u], hi[u]));
                }
            }
        }
    }
}

// ---- tiled general kernel ----------------------------------------------------

struct MoveParams {
    Operand src;
    Operand dst;
    Leading leading;
    uint32_t rows;
    uint32_t cols;
    uint32_t tile_rows;
    uint32_t tile_cols;
    uint32_t elem;        // destination leaf bytes for Copy; unused for casts
    uint64_t items;       // planes * tile_rows * tile_cols
};

__device__ __forceinline__ void store_bytes_masked(
        unsigned char* address, uint4 value, uint32_t valid_bytes) {
    if (valid_bytes >= 16) {
        store_u4(address, value);
        return;
    }
    const uint32_t words[4] = {value.x, value.y, value.z, value.w};
    for (uint32_t b = 0; b < valid_bytes; ++b) {
        address[b] = static_cast<unsigned char>(words[b / 4] >> ((b & 3u) * 8));
    }
}

// One warp per tile. Copy: the tile is 256*elem bytes = elem*16 vectors of 16
// bytes; vector k covers elements [k*16/elem, (k+1)*16/elem) of the tile.
__global__ void __launch_bounds__(kCopyThreads)
copy_tiled_kernel(const MoveParams p) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kCopyWarps + (threadIdx.x >> 5);
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kCopyWarps;
    const uint32_t tile_bytes = kTileSlots * p.elem;
    const uint32_t tile_vectors = tile_bytes / 16;
    const uint32_t per_vector = 16 / p.elem;      // elements per vector (>= 2)
    for (uint64_t item = warp; item < p.items; item += warps) {
        const uint32_t tc = static_cast<uint32_t>(item % p.tile_cols);
        const uint64_t band = item / p.tile_cols;
        const uint32_t tr = static_cast<uint32_t>(band % p.tile_rows);
        const uint64_t index = band / p.tile_rows;
        const uint64_t tile_in_plane = static_cast<uint64_t>(tr) * p.tile_cols + tc;
        const unsigned char* src = p.src.base
                + (operand_plane(p.src, p.leading, index) * p.tile_rows * p.tile_cols
                   + tile_in_plane) * tile_bytes;
        unsigned char* dst = p.dst.base
                + (operand_plane(p.dst, p.leading, index) * p.tile_rows * p.tile_cols
                   + tile_in_plane) * tile_bytes;
        const uint32_t rows_left = p.rows - tr * kTile;
        const uint32_t cols_left = p.cols - tc * kTile;
        for (uint32_t k = lane; k < tile_vectors; k += 32) {
            const uint32_t slot = k * per_vector;
            const uint32_t row = slot / kTile, col = slot % kTile;
            if (row >= rows_left || col >= cols_left) continue;
            const uint32_t valid = min(per_vector, cols_left - col);
            store_bytes_masked(dst + k * 16, load_u4(src + k * 16), valid * p.elem);
        }
    }
}

// One warp per tile; lane L owns 8 elements: BF16 bytes [16L,16L+16) and F32
// bytes [32L,32L+32) of the same tile (row L/2, columns (L%2)*8 .. +7).
template <Move M>
__global__ void __launch_bounds__(kCopyThreads)
cast_tiled_kernel(const MoveParams p) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kCopyWarps + (threadIdx.x >> 5);
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kCopyWarps;
    constexpr uint32_t kSrcTile = M == Move::Bf16ToF32 ? 512u : 1024u;
    constexpr uint32_t kDstTile = M == Move::Bf16ToF32 ? 1024u : 512u;
    const uint32_t row = lane / 2, col = (lane % 2) * 8;
    for (uint64_t item = warp; item < p.items; item += warps) {
        const uint32_t tc = static_cast<uint32_t>(item % p.tile_cols);
        const uint64_t band = item / p.tile_cols;
        const uint32_t tr = static_cast<uint32_t>(band % p.tile_rows);
        const uint64_t index = band / p.tile_rows;
        const uint64_t tile_in_plane = static_cast<uint64_t>(tr) * p.tile_cols + tc;
        const unsigned char* src = p.src.base
                + (operand_plane(p.src, p.leading, index) * p.tile_rows * p.tile_cols
                   + tile_in_plane) * kSrcTile;
        unsigned char* dst = p.dst.base
                + (operand_plane(p.dst, p.leading, index) * p.tile_rows * p.tile_cols
                   + tile_in_plane) * kDstTile;
        const uint32_t rows_left = p.rows - tr * kTile;
        const uint32_t cols_left = p.cols - tc * kTile;
        if (row >= rows_left || col >= cols_left) continue;
        const uint32_t valid = min(8u, cols_left - col);
        if constexpr (M == Move::Bf16ToF32) {
            uint4 lo, hi;
            widen_vector(load_u4(src + lane * 16), &lo, &hi);
            store_bytes_masked(dst + lane * 32, lo, min(valid, 4u) * 4);
            if (valid > 4) store_bytes_masked(dst + lane * 32 + 16, hi, (valid - 4) * 4);
        } else {
            const uint4 lo = load_u4(src + lane * 32);
            const uint4 hi = load_u4(src + lane * 32 + 16);
            store_bytes_masked(dst + lane * 16, narrow_vectors(lo, hi), valid * 2);
        }
    }
}

// ---- host layout <-> tiled ---------------------------------------------------

struct LayoutParams {
    Operand view;
    Leading leading;
    unsigned char* logical;   // row-major payload of the view
    uint32_t rows;
    uint32_t cols;
    uint32_t tile_rows;
    uint32_t tile_cols;
    uint32_t elem;
    uint32_t vector_ok;       // logical rows start 16-byte aligned
    uint64_t items;
};

template <bool TO_TILED>
__global__ void __launch_bounds__(kCopyThreads)
layout_kernel(const LayoutParams p) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kCopyWarps + (threadIdx.x >> 5);
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kCopyWarps;
    const uint32_t tile_bytes = kTileSlots * p.elem;
    const uint32_t tile_vectors = tile_bytes / 16;
    const uint32_t per_vector = 16 / p.elem;
    for (uint64_t item = warp; item < p.items; item += warps) {
        const uint32_t tc = static_cast<uint32_t>(item % p.tile_cols);
        const uint64_t band = item / p.tile_cols;
        const uint32_t tr = static_cast<uint32_t>(band % p.tile_rows);
        const uint64_t index = band / p.tile_rows;
        unsigned char* tile = p.view.base
                + (operand_plane(p.view, p.leading, index) * p.tile_rows * p.tile_cols
                   + static_cast<uint64_t>(tr) * p.tile_cols + tc) * tile_bytes;
        const uint32_t rows_left = p.rows - tr * kTile;
        const uint32_t cols_left = p.cols - tc * kTile;
        for (uint32_t k = lane; k < tile_vectors; k += 32) {
            const uint32_t slot = k * per_vector;
            const uint32_t row = slot / kTile, col = slot % kTile;
            if (row >= rows_left || col >= cols_left) continue;
            const uint32_t valid = min(per_vector, cols_left - col);
            unsigned char* host = p.logical
                    + ((index * p.rows + tr * kTile + row) * static_cast<uint64_t>(p.cols)
                       + tc * kTile + col) * p.elem;
            unsigned char* tiled = tile + k * 16;
            if (p.vector_ok && valid == per_vector) {
                if (TO_TILED) store_u4(tiled, load_u4(host));
                else store_u4(host, load_u4(tiled));
            } else {
                const uint32_t bytes = valid * p.elem;
                for (uint32_t b = 0; b < bytes; ++b) {
                    if (TO_TILED) tiled[b] = host[b];
                    else host[b] = tiled[b];
                }
            }
        }
    }
}

// ---- host dispatch -----------------------------------------------------------

static bool same_shape(const iomb_view& a, const iomb_view& b) {
    if (a.rank != b.rank) return false;
    for (uint32_t i = 0; i < a.rank; ++i) {
        if (a.dims[i] != b.dims[i]) return false;
    }
    return true;
}

// ---- leaves of 2, 4 and 6 bits ------------------------------------------------------
//
// Slots are packed LSB first, so the 16 slots of a tile row are 4, 8 or 12 whole bytes. One
// thread owns one tile row of the tiled side: it replaces the logical columns and keeps the
// bits of the padding columns. The logical (host-layout) payload is one LSB-first bit
// stream over planes, rows and columns (include/iom/tensor.hpp:330-342), so its rows do not
// start on byte boundaries: when it is the destination, one thread owns one payload byte.
struct NarrowParams {
    Operand src;              // tiled source (copy, gather)
    Operand dst;              // tiled destination (copy, scatter)
    Leading leading;
    unsigned char* logical;   // payload (scatter: source, gather: destination)
    uint32_t rows, cols, tile_rows, tile_cols, bits;
    uint32_t dst_row_offset;  // cache_append: source row r lands on destination row offset + r
    uint64_t items;
};

__device__ __forceinline__ uint32_t narrow_bits_at(const unsigned char* base, uint64_t bit, uint32_t bits) {
    const unsigned char* byte = base + (bit >> 3);
    const uint32_t shift = static_cast<uint32_t>(bit & 7u);
    uint32_t value = static_cast<uint32_t>(byte[0]) >> shift;
    if (shift + bits > 8) value |= static_cast<uint32_t>(byte[1]) << (8 - shift);
    return value & ((1u << bits) - 1u);
}

__device__ __forceinline__ uint64_t narrow_slot(const Operand& operand, const Leading& leading,
                                                uint64_t index, uint32_t row, uint32_t col) {
    const uint64_t tile = (operand_plane(operand, leading, index) * operand.tile_rows + row / kTile)
            * operand.tile_cols + col / kTile;
    return tile * kTileSlots + (row % kTile) * kTile + col % kTile;
}

// FROM_LOGICAL: scatter (payload -> tiled), else copy (tiled -> tiled).
template <bool FROM_LOGICAL>
__global__ void __launch_bounds__(kCopyThreads)
narrow_rows_kernel(const NarrowParams p) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kCopyThreads;
    const uint32_t row_bytes = 2 * p.bits;
    for (uint64_t item = static_cast<uint64_t>(blockIdx.x) * kCopyThreads + threadIdx.x; item < p.items;
         item += stride) {
        const uint32_t tc = static_cast<uint32_t>(item % p.tile_cols);
        const uint64_t rest = item / p.tile_cols;
        const uint32_t row = static_cast<uint32_t>(rest % p.rows);
        const uint64_t index = rest / p.rows;
        const uint32_t live = min(kTile, p.cols - tc * kTile);
        unsigned char* out = p.dst.base
                + narrow_slot(p.dst, p.leading, index, row + p.dst_row_offset, tc * kTile) * p.bits / 8;
        unsigned __int128 packed = 0;
        for (uint32_t b = 0; b < row_bytes; ++b) packed |= static_cast<unsigned __int128>(out[b]) << (8 * b);
        for (uint32_t c = 0; c < live; ++c) {
            const uint32_t col = tc * kTile + c;
            uint32_t value;
            if constexpr (FROM_LOGICAL) {
                const uint64_t element = (index * p.rows + row) * p.cols + col;
                value = narrow_bits_at(p.logical, element * p.bits, p.bits);
            } else {
                value = narrow_bits_at(p.src.base, narrow_slot(p.src, p.leading, index, row, col) * p.bits, p.bits);
            }
            const unsigned __int128 mask = static_cast<unsigned __int128>((1u << p.bits) - 1u) << (c * p.bits);
            packed = (packed & ~mask) | (static_cast<unsigned __int128>(value) << (c * p.bits));
        }
        for (uint32_t b = 0; b < row_bytes; ++b) out[b] = static_cast<unsigned char>(packed >> (8 * b));
    }
}

// gather: one thread per payload byte; the bits past the last element are zero.
__global__ void __launch_bounds__(kCopyThreads)
narrow_gather_kernel(const NarrowParams p) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kCopyThreads;
    const uint64_t elements = p.leading.planes * p.rows * p.cols;
    for (uint64_t byte = static_cast<uint64_t>(blockIdx.x) * kCopyThreads + threadIdx.x; byte < p.items;
         byte += stride) {
        const uint64_t first_bit = byte * 8;
        uint32_t assembled = 0;
        for (uint64_t element = first_bit / p.bits; element < elements && element * p.bits < first_bit + 8;
             ++element) {
            const uint32_t col = static_cast<uint32_t>(element % p.cols);
            const uint64_t rest = element / p.cols;
            const uint32_t row = static_cast<uint32_t>(rest % p.rows);
            const uint64_t index = rest / p.rows;
            const uint32_t value = narrow_bits_at(
                    p.src.base, narrow_slot(p.src, p.leading, index, row, col) * p.bits, p.bits);
            const int64_t offset = static_cast<int64_t>(element * p.bits) - static_cast<int64_t>(first_bit);
            assembled |= offset >= 0 ? value << offset : value >> (-offset);
        }
        p.logical[byte] = static_cast<unsigned char>(assembled);
    }
}

static bool narrow_leaf(uint32_t bits) { return bits == 2 || bits == 4 || bits == 6; }

// cache_append of a 2-, 4- or 6-bit leaf: the row copy of narrow_rows_kernel with the
// destination rows shifted by `a` (both views validated by the caller).
int narrow_append(const iomb_view& source, const ViewFacts& fs, const iomb_view& destination,
                  const ViewFacts& fd, uint64_t a, cudaStream_t stream) {
    if (!narrow_leaf(fs.bits)) return fail(IOMB_ERR_UNSUPPORTED, "cache_append: leaf width is not 2, 4 or 6 bits");
    NarrowParams n{};
    uint64_t strides[2][kMaxLead] = {};
    for (uint32_t axis = 0; axis < fs.leading; ++axis) {
        strides[0][axis] = source.plane_strides[axis];
        strides[1][axis] = destination.plane_strides[axis];
    }
    collapse_leading(fs.leading, source.dims, strides, 2, &n.leading);
    n.src = make_operand(source, fs, strides[0], n.leading, false, false);
    n.dst = make_operand(destination, fd, strides[1], n.leading, false, false);
    n.rows = static_cast<uint32_t>(fs.rows);
    n.cols = static_cast<uint32_t>(fs.cols);
    n.tile_rows = static_cast<uint32_t>(fs.tile_rows);
    n.tile_cols = static_cast<uint32_t>(fs.tile_cols);
    n.bits = fs.bits;
    n.dst_row_offset = static_cast<uint32_t>(a);
    n.items = n.leading.planes * fs.rows * fs.tile_cols;
    narrow_rows_kernel<false><<<grid_for((n.items + kCopyThreads - 1) / kCopyThreads, 8), kCopyThreads, 0,
                                stream>>>(n);
    return check_launch("cache_append launch");
}

static int move_dispatch(const iomb_view* source, const iomb_view* destination, Move move,
                         void* stream) {
    ViewFacts fs{}, fd{};
    int status = check_view(source, "copy source", &fs);
    if (status == IOMB_OK) status = check_view(destination, "copy destination", &fd);
    if (status != IOMB_OK) return status;
    if (!same_shape(*source, *destination)) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "copy views must have identical shape");
    }
    if (fd.rows > 0xFFFFFFFFull || fd.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "copy: matrix extent exceeds the kernel limit");
    }
    MoveParams p{};
    uint64_t strides[2][kMaxLead] = {};
    for (uint32_t axis = 0; axis < fs.leading; ++axis) {
        strides[0][axis] = source->plane_strides[axis];
        strides[1][axis] = destination->plane_strides[axis];
    }
    collapse_leading(fs.leading, source->dims, strides, 2, &p.leading);
    p.src = make_operand(*source, fs, strides[0], p.leading, false, false);
    p.dst = make_operand(*destination, fd, strides[1], p.leading, false, false);
    p.rows = static_cast<uint32_t>(fd.rows);
    p.cols = static_cast<uint32_t>(fd.cols);
    p.tile_rows = static_cast<uint32_t>(fd.tile_rows);
    p.tile_cols = static_cast<uint32_t>(fd.tile_cols);
    p.elem = fd.bytes;
    p.items = p.leading.planes * fd.tile_rows * fd.tile_cols;
    const bool linear = p.leading.contiguous && fd.rows % kTile == 0 && fd.cols % kTile == 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (linear) {
        const unsigned char* src = p.src.base + source->plane_offset * fs.plane_bytes;
        unsigned char* dst = p.dst.base + destination->plane_offset * fd.plane_bytes;
        if (move == Move::Copy) {
            const uint64_t vectors = p.leading.planes * fd.plane_bytes / 16;
            const uint64_t per_cta = static_cast<uint64_t>(kCopyThreads) * kCopyUnroll;
            copy_linear_kernel<<<grid_one_shot((vectors + per_cta - 1) / per_cta), kCopyThreads, 0, s>>>(
                    reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), vectors);
        } else {
            const uint64_t groups = p.leading.planes * fd.tile_rows * fd.tile_cols * kTileSlots / 8;
            const unsigned grid = grid_one_shot((groups + kCopyThreads * 4 - 1) / (kCopyThreads * 4));
            if (move == Move::Bf16ToF32) {
                cast_linear_kernel<Move::Bf16ToF32><<<grid, kCopyThreads, 0, s>>>(
                        reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), groups);
            } else {
                cast_linear_kernel<Move::F32ToBf16><<<grid, kCopyThreads, 0, s>>>(
                        reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), groups);
            }
        }
    } else if (fd.bytes == 0) {
        NarrowParams n{};
        n.src = p.src;
        n.dst = p.dst;
        n.leading = p.leading;
        n.rows = p.rows;
        n.cols = p.cols;
        n.tile_rows = p.tile_rows;
        n.tile_cols = p.tile_cols;
        n.bits = fd.bits;
        n.items = p.leading.planes * fd.rows * fd.tile_cols;
        narrow_rows_kernel<false><<<grid_for((n.items + kCopyThreads - 1) / kCopyThreads, 8), kCopyThreads, 0, s>>>(n);
    } else {
        const unsigned grid = grid_one_shot((p.items + kCopyWarps - 1) / kCopyWarps);
        if (move == Move::Copy) {
            copy_tiled_kernel<<<grid, kCopyThreads, 0, s>>>(p);
        } else if (move == Move::Bf16ToF32) {
            cast_tiled_kernel<Move::Bf16ToF32><<<grid, kCopyThreads, 0, s>>>(p);
        } else {
            cast_tiled_kernel<Move::F32ToBf16><<<grid, kCopyThreads, 0, s>>>(p);
        }
    }
    return check_launch("copy launch");
}

static int layout_dispatch(const iomb_view* view, void* logical, bool to_tiled, void* stream) {
    ViewFacts f{};
    const int status = check_view(view, to_tiled ? "scatter destination" : "gather source", &f);
    if (status != IOMB_OK) return status;
    if (logical == nullptr) return fail(IOMB_ERR_INVALID_ARGUMENT, "staging buffer is null");
    if (f.bytes == 0 && !narrow_leaf(f.bits)) {
        return fail(IOMB_ERR_UNSUPPORTED, "host transfer: leaf width is neither a byte multiple nor 2, 4 or 6 bits");
    }
    if (f.rows > 0xFFFFFFFFull || f.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "host transfer: matrix extent exceeds the kernel limit");
    }
    if (f.bytes == 0) {
        NarrowParams n{};
        uint64_t narrow_strides[1][kMaxLead] = {};
        for (uint32_t axis = 0; axis < f.leading; ++axis) narrow_strides[0][axis] = view->plane_strides[axis];
        collapse_leading(f.leading, view->dims, narrow_strides, 1, &n.leading);
        n.src = make_operand(*view, f, narrow_strides[0], n.leading, false, false);
        n.dst = n.src;
        n.logical = static_cast<unsigned char*>(logical);
        n.rows = static_cast<uint32_t>(f.rows);
        n.cols = static_cast<uint32_t>(f.cols);
        n.tile_rows = static_cast<uint32_t>(f.tile_rows);
        n.tile_cols = static_cast<uint32_t>(f.tile_cols);
        n.bits = f.bits;
        cudaStream_t narrow_stream = static_cast<cudaStream_t>(stream);
        if (to_tiled) {
            n.items = n.leading.planes * f.rows * f.tile_cols;
            narrow_rows_kernel<true><<<grid_for((n.items + kCopyThreads - 1) / kCopyThreads, 8), kCopyThreads, 0,
                                       narrow_stream>>>(n);
        } else {
            n.items = (n.leading.planes * f.rows * f.cols * f.bits + 7) / 8;
            narrow_gather_kernel<<<grid_for((n.items + kCopyThreads - 1) / kCopyThreads, 8), kCopyThreads, 0,
                                   narrow_stream>>>(n);
        }
        return check_launch("host transfer launch");
    }
    LayoutParams p{};
    uint64_t strides[1][kMaxLead] = {};
    for (uint32_t axis = 0; axis < f.leading; ++axis) strides[0][axis] = view->plane_strides[axis];
    // The logical payload enumerates planes in the view's own leading order, so
    // the axes are kept as they are (a merge would not change the order either).
    collapse_leading(f.leading, view->dims, strides, 1, &p.leading);
    p.view = make_operand(*view, f, strides[0], p.leading, false, false);
    p.logical = static_cast<unsigned char*>(logical);
    p.rows = static_cast<uint32_t>(f.rows);
    p.cols = static_cast<uint32_t>(f.cols);
    p.tile_rows = static_cast<uint32_t>(f.tile_rows);
    p.tile_cols = static_cast<uint32_t>(f.tile_cols);
    p.elem = f.bytes;
    p.vector_ok = (reinterpret_cast<uintptr_t>(logical) % 16 == 0
                   && (f.cols * f.bytes) % 16 == 0) ? 1u : 0u;
    p.items = p.leading.planes * f.tile_rows * f.tile_cols;
    const unsigned grid = grid_for((p.items + kCopyWarps - 1) / kCopyWarps, 8);
    if (to_tiled) {
        layout_kernel<true><<<grid, kCopyThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    } else {
        layout_kernel<false><<<grid, kCopyThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    }
    return check_launch("host transfer launch");
}

}  // namespace iomb

extern "C" int iomb_copy(const iomb_view* source, const iomb_view* destination, void* stream) {
    using namespace iomb;
    if (source != nullptr && destination != nullptr) {
        if (source->dtype != destination->dtype) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "copy views must have identical leaf type");
        }
        const uint32_t bits = iomb_dtype_bits(source->dtype);
        if (bits != 0 && bits % 8 != 0 && !narrow_leaf(bits)) {
            return fail(IOMB_ERR_UNSUPPORTED, "copy: leaf width is neither a byte multiple nor 2, 4 or 6 bits");
        }
    }
    ViewFacts fs{}, fd{};
    int status = check_view(source, "copy source", &fs);
    if (status == IOMB_OK) status = check_view(destination, "copy destination", &fd);
    if (status != IOMB_OK) return status;
    // An identical window is an accepted no-op (src/device_ops_copy.cpp:28-37).
    if (same_window(*source, *destination)) return IOMB_OK;
    return move_dispatch(source, destination, Move::Copy, stream);
}

extern "C" int iomb_cast(const iomb_view* source, const iomb_view* destination, void* stream) {
    using namespace iomb;
    if (source == nullptr || destination == nullptr) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "cast: view is null");
    }
    if (source->dtype == IOMB_BF16 && destination->dtype == IOMB_F32) {
        return move_dispatch(source, destination, Move::Bf16ToF32, stream);
    }
    if (source->dtype == IOMB_F32 && destination->dtype == IOMB_BF16) {
        return move_dispatch(source, destination, Move::F32ToBf16, stream);
    }
    return fail(IOMB_ERR_UNSUPPORTED, "cast: only BF16<->F32 is implemented");
}

extern "C" int iomb_scatter(const iomb_view* destination, const void* staging, void* stream) {
    return iomb::layout_dispatch(destination, const_cast<void*>(staging), true, stream);
}

extern "C" int iomb_gather(const iomb_view* source, void* staging, void* stream) {
    return iomb::layout_dispatch(source, staging, false, stream);
}
