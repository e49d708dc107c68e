// Row movers on tiled storage: embedding lookup and KV-cache append.
//
// A logical row of F elements is F/16 pieces of one in-tile row (16 elements)
// at a one-tile stride. Both operations copy whole rows bit for bit as 16-byte
// vectors, masking the feature tail; the work is cut by tiles, not by rows, so
// that one side of every move is a whole contiguous tile.
//
// Replaces embedding_word_kernel (src/shared/standard_tiled_embedding.inl:117-199)
// and cache_append_kernel (src/cuda/copy.cu:135-214). The reference append
// kernel visits every word of every destination plane to append one row; this
// one touches the appended rows only.
#include "host.hpp"

namespace iomb {

constexpr int kRowThreads = 256;
constexpr int kRowWarps = kRowThreads / 32;
// Neighbouring tiles of a band one warp moves at once (template parameter TILES): more
// bytes in flight per decoded id when the request has items to spare, fewer when it is a
// decode step that has to be spread over the SMs.
__host__ inline uint32_t tiles_per_item(uint64_t bands, uint64_t tile_cols, uint32_t widest) {
    const uint64_t warps = static_cast<uint64_t>(sm_count() > 0 ? sm_count() : 148) * 32;
    for (uint32_t tiles = widest; tiles > 1; tiles /= 2) {
        if (bands * ((tile_cols + tiles - 1) / tiles) >= 2 * warps && tile_cols >= tiles) return tiles;
    }
    return 1;
}

struct RowGeometry {
    uint32_t elem;          // leaf bytes
    uint32_t cols;          // logical features
    uint32_t tile_cols;
    uint32_t row_vectors;   // tile_cols * (16*elem/16)
};

// Stores one 16-byte vector, or only its first `valid` elements at the feature tail.
template <bool STREAM = false>
__device__ __forceinline__ void store_row_vector(unsigned char* address, uint4 value,
                                                 uint32_t valid, uint32_t per_vector,
                                                 uint32_t elem) {
    if (valid >= per_vector) {
        if constexpr (STREAM) store_u4_stream(address, value); else store_u4(address, value);
        return;
    }
    const uint32_t words[4] = {value.x, value.y, value.z, value.w};
    const uint32_t bytes = valid * elem;
    for (uint32_t b = 0; b < bytes; ++b) {
        address[b] = static_cast<unsigned char>(words[b / 4] >> ((b & 3u) * 8));
    }
}

// Byte address of tile (row / 16, tile_col) of `plane`, at in-tile row row % 16.
__device__ __forceinline__ unsigned char* piece_address(
        const Operand& operand, uint64_t plane, uint64_t row, uint32_t tile_col, uint32_t elem) {
    const uint64_t tile = (plane * operand.tile_rows + row / kTile) * operand.tile_cols + tile_col;
    return operand.base + tile * kTileSlots * elem + (row % kTile) * kTile * elem;
}

// Both movers give one warp one 16x16 tile: the tile of the result (embedding) or
// of the source (append). Its 16 in-tile rows are 16 consecutive row pieces, so a
// warp reads or writes whole contiguous tiles; the other side of the move is, per
// row, one piece of 16 elements somewhere else (a table row, a shifted cache row).

// ---- embedding ---------------------------------------------------------------

struct EmbeddingParams {
    Operand table;      // rank two: plane0 is the selected table plane
    Operand indices;
    Operand out;
    Leading leading;    // leading space of indices/out
    RowGeometry row;
    uint32_t run;             // R: rows per plane
    uint32_t run_tiles;       // ceil(R / 16)
    uint32_t index_bits;      // 2, 4, 8, 16, 32 or 64
    uint32_t index_signed;
    uint64_t vocabulary;
    uint64_t items;           // planes * run_tiles * ceil(tile_cols / TILES)
    uint32_t* status;
};

// indices[b, 0, r]: tile column r / 16, in-tile row 0, column r % 16 of the index plane;
// slots are packed LSB first, so an id of 2 or 4 bits never straddles a byte. Compared at
// full width against the vocabulary (src/shared/standard_tiled_embedding.inl:160-172):
// false for a negative id or one at or beyond the table's rows.
__device__ __forceinline__ bool read_index(const EmbeddingParams& p, uint64_t index_plane,
                                           uint32_t r, uint64_t* id_out) {
    const uint64_t slot = ((index_plane * p.indices.tile_rows) * p.indices.tile_cols + r / kTile)
                    * static_cast<uint64_t>(kTileSlots)
            + r % kTile;
    const uint64_t bit = slot * p.index_bits;
    const unsigned char* address = p.indices.base + (bit >> 3);
    uint64_t id = 0;
    switch (p.index_bits) {
        case 2: id = (*address >> (bit & 7u)) & 0x3u; break;
        case 4: id = (*address >> (bit & 7u)) & 0xFu; break;
        case 8: id = *address; break;
        case 16: id = *reinterpret_cast<const uint16_t*>(address); break;
        case 32: id = *reinterpret_cast<const uint32_t*>(address); break;
        default: id = *reinterpret_cast<const uint64_t*>(address); break;
    }
    const bool negative = p.index_signed && ((id >> (p.index_bits - 1)) & 1u);
    *id_out = id;
    return !negative && id < p.vocabulary;
}

template <uint32_t kTilesPerItem>
__global__ void __launch_bounds__(kRowThreads)
embedding_kernel(const EmbeddingParams p) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5);
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kRowWarps;
    const uint32_t elem = p.row.elem;
    // The table is read again and again while the output streams through L2 once: the table's
    // lines are asked to stay, the output's to leave first.
    const uint64_t keep = l2_keep_policy();
    const uint32_t vectors_per_row = elem;                 // (16 * elem) / 16
    const uint32_t per_vector = 16 / elem;
    const uint32_t tile_vectors = kTile * vectors_per_row;
    const uint32_t groups = (p.row.tile_cols + kTilesPerItem - 1) / kTilesPerItem;
    for (uint64_t item = warp; item < p.items; item += warps) {
        // item = ((index * run_tiles) + tr) * groups + group: kTilesPerItem neighbouring
        // tiles of one band share the band's ids, decoded once per lane.
        const uint32_t group = static_cast<uint32_t>(item % groups);
        const uint64_t rest = item / groups;
        const uint32_t tr = static_cast<uint32_t>(rest % p.run_tiles);
        const uint64_t index = rest / p.run_tiles;
        const uint64_t index_plane = operand_plane(p.indices, p.leading, index);
        const uint64_t out_plane = operand_plane(p.out, p.leading, index);
        const uint32_t first_tc = group * kTilesPerItem;
        const uint32_t tiles = min(kTilesPerItem, p.row.tile_cols - first_tc);
        for (uint32_t k = lane; k < tile_vectors; k += 32) {
            const uint32_t row_in_tile = k / vectors_per_row;
            const uint32_t r = tr * kTile + row_in_tile;
            if (r >= p.run) continue;
            const uint32_t cv = k % vectors_per_row;
            // indices[b, 0, r]: tile column r / 16, in-tile row 0, column r % 16.
            uint64_t id = 0;
            if (!read_index(p, index_plane, r, &id)) {
                // Never form a table address from an invalid id
                // (standard_tiled_embedding.inl:167-172); one report per row.
                if (group == 0 && cv == 0) atomicOr(p.status, 1u);
                continue;
            }
            const unsigned char* src = piece_address(p.table, p.table.plane0, id, first_tc, elem) + cv * 16;
            unsigned char* dst = piece_address(p.out, out_plane, r, first_tc, elem) + cv * 16;
            const size_t tile_bytes = static_cast<size_t>(kTileSlots) * elem;
            uint4 value[kTilesPerItem];
#pragma unroll
            for (uint32_t t = 0; t < kTilesPerItem; ++t) {
                if (t < tiles) value[t] = load_u4_keep(src + t * tile_bytes, keep);
            }
#pragma unroll
            for (uint32_t t = 0; t < kTilesPerItem; ++t) {
                if (t >= tiles) continue;
                const uint32_t col = (first_tc + t) * kTile + cv * per_vector;
                if (col >= p.row.cols) continue;
                store_row_vector<true>(dst + t * tile_bytes, value[t], min(per_vector, p.row.cols - col),
                                 per_vector, elem);
            }
        }
    }
}

// ---- cache append --------------------------------------------------------------

struct AppendParams {
    Operand src;
    Operand dst;
    Leading leading;
    RowGeometry row;
    uint32_t rows;              // R: appended rows per plane
    uint32_t row_tiles;         // ceil(R / 16)
    uint64_t dst_rows;          // C: cache length
    uint64_t a;                 // scalar offset (positions == nullptr)
    const uint32_t* positions;  // per index of the first leading axis, or nullptr
    uint64_t planes_per_batch;  // logical planes per index of the first leading axis
    uint64_t items;             // planes * row_tiles * ceil(tile_cols / TILES)
    uint32_t* status;           // batched only
};

template <uint32_t kTilesPerItem>
__global__ void __launch_bounds__(kRowThreads)
cache_append_kernel(const AppendParams p) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5);
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kRowWarps;
    const uint32_t elem = p.row.elem;
    const uint32_t vectors_per_row = elem;
    const uint32_t per_vector = 16 / elem;
    const uint32_t tile_vectors = kTile * vectors_per_row;
    const uint32_t groups = (p.row.tile_cols + kTilesPerItem - 1) / kTilesPerItem;
    for (uint64_t item = warp; item < p.items; item += warps) {
        const uint32_t group = static_cast<uint32_t>(item % groups);
        const uint64_t rest = item / groups;
        const uint32_t tr = static_cast<uint32_t>(rest % p.row_tiles);
        const uint64_t index = rest / p.row_tiles;
        uint64_t a = p.a;
        if (p.positions != nullptr) {
            a = p.positions[index / p.planes_per_batch];
            if (a > p.dst_rows || p.rows > p.dst_rows - a) {
                if (lane == 0 && group == 0 && tr == 0) atomicOr(p.status, 1u);
                continue;
            }
        }
        const uint64_t src_plane = operand_plane(p.src, p.leading, index);
        const uint64_t dst_plane = operand_plane(p.dst, p.leading, index);
        const uint32_t first_tc = group * kTilesPerItem;
        const uint32_t tiles = min(kTilesPerItem, p.row.tile_cols - first_tc);
        const size_t tile_bytes = static_cast<size_t>(kTileSlots) * elem;
        for (uint32_t k = lane; k < tile_vectors; k += 32) {
            const uint32_t row_in_tile = k / vectors_per_row;
            const uint32_t r = tr * kTile + row_in_tile;
            if (r >= p.rows) continue;
            const uint32_t cv = k % vectors_per_row;
            const unsigned char* src = piece_address(p.src, src_plane, r, first_tc, elem) + cv * 16;
            unsigned char* dst = piece_address(p.dst, dst_plane, a + r, first_tc, elem) + cv * 16;
            uint4 value[kTilesPerItem];
#pragma unroll
            for (uint32_t t = 0; t < kTilesPerItem; ++t) {
                if (t < tiles) value[t] = load_u4(src + t * tile_bytes);
            }
#pragma unroll
            for (uint32_t t = 0; t < kTilesPerItem; ++t) {
                if (t >= tiles) continue;
                const uint32_t col = (first_tc + t) * kTile + cv * per_vector;
                if (col >= p.row.cols) continue;
                store_row_vector(dst + t * tile_bytes, value[t], min(per_vector, p.row.cols - col),
                                 per_vector, elem);
            }
        }
    }
}

// ---- host dispatch ---------------------------------------------------------------

static RowGeometry row_geometry(const ViewFacts& f) {
    RowGeometry g{};
    g.elem = f.bytes;
    g.cols = static_cast<uint32_t>(f.cols);
    g.tile_cols = static_cast<uint32_t>(f.tile_cols);
    g.row_vectors = g.tile_cols * g.elem;
    return g;
}

static int append_dispatch(const iomb_view* source, const iomb_view* destination, uint64_t a,
                           const uint32_t* positions, uint32_t* status, void* stream) {
    ViewFacts fs{}, fd{};
    int rc = check_view(source, "cache_append source", &fs);
    if (rc == IOMB_OK) rc = check_view(destination, "cache_append destination", &fd);
    if (rc != IOMB_OK) return rc;
    // Admission of validate_cache_append (src/device_ops_cache_append.cpp:157-269).
    if (source->rank < 3 || source->rank != destination->rank) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append requires equal ranks of three through eight");
    }
    for (uint32_t i = 0; i + 2 < source->rank; ++i) {
        if (source->dims[i] != destination->dims[i]) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append leading and head extents differ");
        }
    }
    if (fs.cols != fd.cols) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append feature widths differ");
    }
    if (source->dtype != destination->dtype) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append encodings differ");
    }
    if (positions == nullptr) {
        if (a > fd.rows || fs.rows > fd.rows - a) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append rows exceed the cache length");
        }
    } else {
        if (status == nullptr) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append_batched: status is null");
        }
        if (fs.rows > fd.rows) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append rows exceed the cache length");
        }
    }
    if (storage_overlaps(*source, fs, *destination, fd)) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append source and destination storage overlap");
    }
    if (fs.rows > 0xFFFFFFFFull || fs.cols > 0xFFFFFFFFull || fd.rows > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "cache_append: matrix extent exceeds the kernel limit");
    }
    if (fs.bytes == 0) {
        if (positions != nullptr) {
            return fail(IOMB_ERR_UNSUPPORTED, "cache_append_batched: sub-byte leaves are not implemented");
        }
        return narrow_append(*source, fs, *destination, fd, a, static_cast<cudaStream_t>(stream));
    }
    AppendParams p{};
    uint64_t strides[2][kMaxLead] = {};
    for (uint32_t axis = 0; axis < fs.leading; ++axis) {
        strides[0][axis] = source->plane_strides[axis];
        strides[1][axis] = destination->plane_strides[axis];
    }
    if (positions == nullptr) {
        collapse_leading(fs.leading, source->dims, strides, 2, &p.leading);
    } else {
        // Keep the leading axes as they are so the first axis stays addressable.
        p.leading.count = fs.leading;
        p.leading.planes = fs.planes;
        p.leading.contiguous = 0;
        for (uint32_t axis = 0; axis < kMaxLead; ++axis) {
            p.leading.dims[axis] = axis < fs.leading ? source->dims[axis] : 1;
        }
    }
    p.src = make_operand(*source, fs, strides[0], p.leading, false, false);
    p.dst = make_operand(*destination, fd, strides[1], p.leading, false, false);
    p.row = row_geometry(fs);
    p.rows = static_cast<uint32_t>(fs.rows);
    p.dst_rows = fd.rows;
    p.a = a;
    p.positions = positions;
    p.planes_per_batch = fs.planes / source->dims[0];
    p.row_tiles = static_cast<uint32_t>(fs.tile_rows);
    const uint32_t tiles = tiles_per_item(fs.planes * fs.tile_rows, fs.tile_cols, 4);
    p.items = fs.planes * fs.tile_rows * ((fs.tile_cols + tiles - 1) / tiles);
    p.status = status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (positions != nullptr) {
        if (cudaMemsetAsync(status, 0, sizeof(uint32_t), s) != cudaSuccess) {
            return check_launch("cache_append status reset");
        }
    }
    const unsigned grid = grid_one_shot((p.items + kRowWarps - 1) / kRowWarps);
    switch (tiles) {
        case 4: cache_append_kernel<4><<<grid, kRowThreads, 0, s>>>(p); break;
        case 2: cache_append_kernel<2><<<grid, kRowThreads, 0, s>>>(p); break;
        default: cache_append_kernel<1><<<grid, kRowThreads, 0, s>>>(p); break;
    }
    return check_launch("cache_append launch");
}

// Payload leaves of 2, 4 and 6 bits: one thread per (plane, output row, tile column) moves
// the 4, 8 or 12 bytes of one tile row; in the last tile column only the logical columns are
// replaced, so the bits of padding slots survive. Ids are read and checked as above.
__global__ void __launch_bounds__(kRowThreads)
embedding_narrow_kernel(const EmbeddingParams p, uint32_t bits, uint32_t cols, uint64_t items) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kRowThreads;
    const uint32_t row_bytes = 2 * bits;
    const uint32_t tile_cols = p.out.tile_cols;
    for (uint64_t item = static_cast<uint64_t>(blockIdx.x) * kRowThreads + threadIdx.x; item < items;
         item += stride) {
        const uint32_t tc = static_cast<uint32_t>(item % tile_cols);
        const uint64_t rest = item / tile_cols;
        const uint32_t r = static_cast<uint32_t>(rest % p.run);
        const uint64_t index = rest / p.run;
        uint64_t id = 0;
        if (!read_index(p, operand_plane(p.indices, p.leading, index), r, &id)) {
            if (tc == 0) atomicOr(p.status, 1u);
            continue;
        }
        const uint64_t src_tile = (p.table.plane0 * p.table.tile_rows + id / kTile) * p.table.tile_cols + tc;
        const uint64_t dst_tile = (operand_plane(p.out, p.leading, index) * p.out.tile_rows + r / kTile)
                * p.out.tile_cols + tc;
        const unsigned char* src = p.table.base + (src_tile * kTileSlots + (id % kTile) * kTile) * bits / 8;
        unsigned char* dst = p.out.base + (dst_tile * kTileSlots + (r % kTile) * kTile) * bits / 8;
        const uint32_t live_bits = min(kTile, cols - tc * kTile) * bits;
        for (uint32_t b = 0; b < row_bytes; ++b) {
            if (8 * b >= live_bits) break;
            const uint32_t keep = live_bits - 8 * b >= 8 ? 0u : 0xffu << (live_bits - 8 * b);   // padding bits
            dst[b] = static_cast<unsigned char>((src[b] & ~keep) | (dst[b] & keep));
        }
    }
}

}  // namespace iomb

extern "C" int iomb_embedding(const iomb_view* table, const iomb_view* indices,
                              const iomb_view* out, uint32_t* status, void* stream) {
    using namespace iomb;
    ViewFacts ft{}, fi{}, fo{};
    int rc = check_view(table, "embedding table", &ft);
    if (rc == IOMB_OK) rc = check_view(indices, "embedding indices", &fi);
    if (rc == IOMB_OK) rc = check_view(out, "embedding out", &fo);
    if (rc != IOMB_OK) return rc;
    // Shape structure of validate_embedding (src/device_ops_embedding.cpp:93-162).
    if (table->rank != 2) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "embedding table must have rank two");
    }
    if (indices->rank != out->rank) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "embedding indices and out ranks differ");
    }
    for (uint32_t i = 0; i + 2 < out->rank; ++i) {
        if (indices->dims[i] != out->dims[i]) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "embedding leading extents differ");
        }
    }
    if (fi.rows != 1 || fi.cols != fo.rows || fo.cols != ft.cols) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "embedding shapes must be E[V,F], I[...,1,R], O[...,R,F]");
    }
    if (table->dtype != out->dtype) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "embedding table and out encodings differ");
    }
    if (storage_overlaps(*out, fo, *table, ft) || storage_overlaps(*out, fo, *indices, fi)
            || out->base == table->base || out->base == indices->base) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "embedding output aliases an input");
    }
    if (status == nullptr) {
        return fail(IOMB_ERR_INVALID_ARGUMENT, "embedding: status is null");
    }
    bool index_signed = false;
    switch (indices->dtype) {
        case IOMB_I2: case IOMB_I4:
        case IOMB_I8: case IOMB_I16: case IOMB_I32: case IOMB_I64: index_signed = true; break;
        case IOMB_U2: case IOMB_U4:
        case IOMB_U8: case IOMB_U16: case IOMB_U32: case IOMB_U64: break;
        default:
            return fail(IOMB_ERR_UNSUPPORTED, "embedding: index leaf is not integral");
    }
    if (fo.rows > 0xFFFFFFFFull || fo.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "embedding: matrix extent exceeds the kernel limit");
    }
    const bool narrow_payload = ft.bytes == 0;
    EmbeddingParams p{};
    uint64_t strides[2][kMaxLead] = {};
    for (uint32_t axis = 0; axis < fo.leading; ++axis) {
        strides[0][axis] = indices->plane_strides[axis];
        strides[1][axis] = out->plane_strides[axis];
    }
    collapse_leading(fo.leading, out->dims, strides, 2, &p.leading);
    p.indices = make_operand(*indices, fi, strides[0], p.leading, false, false);
    p.out = make_operand(*out, fo, strides[1], p.leading, false, false);
    Leading none{};
    none.planes = 1;
    p.table = make_operand(*table, ft, strides[0], none, false, false);
    if (!narrow_payload) p.row = row_geometry(ft);
    p.run = static_cast<uint32_t>(fo.rows);
    p.index_bits = fi.bits;
    p.index_signed = index_signed ? 1u : 0u;
    p.vocabulary = ft.rows;
    p.run_tiles = static_cast<uint32_t>(fo.tile_rows);
    const uint32_t tiles = tiles_per_item(p.leading.planes * fo.tile_rows, fo.tile_cols, 8);
    p.items = p.leading.planes * fo.tile_rows * ((fo.tile_cols + tiles - 1) / tiles);
    p.status = status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Reset in queue order, as the reference does before its kernel
    // (src/shared/gpu_queue_operations.inl:899-914).
    if (cudaMemsetAsync(status, 0, sizeof(uint32_t), s) != cudaSuccess) {
        return check_launch("embedding status reset");
    }
    if (narrow_payload) {
        const uint64_t items = p.leading.planes * fo.rows * fo.tile_cols;
        embedding_narrow_kernel<<<grid_for((items + kRowThreads - 1) / kRowThreads, 8), kRowThreads, 0, s>>>(
                p, ft.bits, static_cast<uint32_t>(fo.cols), items);
        return check_launch("embedding launch");
    }
    const unsigned grid = grid_one_shot((p.items + kRowWarps - 1) / kRowWarps);
    switch (tiles) {
        case 8: embedding_kernel<8><<<grid, kRowThreads, 0, s>>>(p); break;
        case 4: embedding_kernel<4><<<grid, kRowThreads, 0, s>>>(p); break;
        case 2: embedding_kernel<2><<<grid, kRowThreads, 0, s>>>(p); break;
        default: embedding_kernel<1><<<grid, kRowThreads, 0, s>>>(p); break;
    }
    return check_launch("embedding launch");
}

extern "C" int iomb_cache_append(const iomb_view* source, const iomb_view* destination,
                                 uint64_t a, void* stream) {
    return iomb::append_dispatch(source, destination, a, nullptr, nullptr, stream);
}

extern "C" int iomb_cache_append_batched(const iomb_view* source, const iomb_view* destination,
                                         const uint32_t* positions, uint32_t* status,
                                         void* stream) {
    if (positions == nullptr) {
        return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "cache_append_batched: positions is null");
    }
    return iomb::append_dispatch(source, destination, 0, positions, status, stream);
}
