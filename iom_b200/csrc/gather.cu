// Row movers on tiled storage: embedding lookup and KV-cache append.
//
// A logical row of F elements is F/16 pieces of one in-tile row (16 elements)
// at a one-tile stride. Both operations copy whole rows bit for bit, so they
// share one device routine that moves a row as 16-byte vectors and masks the
// feature tail.
//
// Replaces embedding_word_kernel (src/shared/standard_tiled_embedding.inl:117-199)
// and cache_append_kernel (src/cuda/copy.cu:135-214). The reference append
// kernel visits every word of every destination plane to append one row; this
// one touches the appended rows only.
#include "host.hpp"

namespace iomb {

constexpr int kRowThreads = 128;

struct RowGeometry {
    uint32_t elem;          // leaf bytes
    uint32_t cols;          // logical features
    uint32_t tile_cols;
    uint32_t row_vectors;   // tile_cols * (16*elem/16)
};

// Moves vectors [first, first+count) of one logical row.
__device__ __forceinline__ void move_row_vectors(
        const unsigned char* src_row, unsigned char* dst_row, const RowGeometry& g,
        uint32_t vector) {
    const uint32_t vectors_per_piece = g.elem;            // (16*elem)/16
    const uint32_t per_vector = 16 / g.elem;
    const uint32_t tile = vector / vectors_per_piece;
    const uint32_t cv = vector % vectors_per_piece;
    const uint32_t col = tile * kTile + cv * per_vector;
    if (col >= g.cols) return;
    const size_t offset = static_cast<size_t>(tile) * kTileSlots * g.elem + cv * 16;
    const uint32_t valid = min(per_vector, g.cols - col);
    const uint4 value = load_u4(src_row + offset);
    if (valid == per_vector) {
        store_u4(dst_row + offset, value);
    } else {
        const uint32_t words[4] = {value.x, value.y, value.z, value.w};
        const uint32_t bytes = valid * g.elem;
        for (uint32_t b = 0; b < bytes; ++b) {
            dst_row[offset + b] = static_cast<unsigned char>(words[b / 4] >> ((b & 3u) * 8));
        }
    }
}

// Byte address of in-tile row `row` of tile column 0 in (plane, row / 16).
__device__ __forceinline__ unsigned char* row_address(
        const Operand& operand, uint64_t plane, uint64_t row, uint32_t elem) {
    const uint64_t tile = (plane * operand.tile_rows + row / kTile) * operand.tile_cols;
    return operand.base + tile * kTileSlots * elem + (row % kTile) * kTile * elem;
}

// ---- embedding ---------------------------------------------------------------

struct EmbeddingParams {
    Operand table;      // rank two: plane0 is the selected table plane
    Operand indices;
    Operand out;
    Leading leading;    // leading space of indices/out
    RowGeometry row;
    uint32_t run;             // R: rows per plane
    uint32_t index_bytes;     // 1, 2, 4 or 8
    uint32_t index_signed;
    uint64_t vocabulary;
    uint64_t total_rows;      // planes * run
    uint32_t chunks;          // vector chunks per row
    uint32_t* status;
};

__global__ void __launch_bounds__(kRowThreads)
embedding_kernel(const EmbeddingParams p) {
    const uint64_t items = p.total_rows * p.chunks;
    for (uint64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t chunk = static_cast<uint32_t>(item % p.chunks);
        const uint64_t global_row = item / p.chunks;
        const uint32_t r = static_cast<uint32_t>(global_row % p.run);
        const uint64_t index = global_row / p.run;
        // indices[b, 0, r]: tile column r / 16, in-tile row 0, column r % 16.
        const uint64_t index_plane = operand_plane(p.indices, p.leading, index);
        const unsigned char* id_address = p.indices.base
                + ((index_plane * p.indices.tile_rows) * p.indices.tile_cols + r / kTile)
                        * static_cast<uint64_t>(kTileSlots) * p.index_bytes
                + (r % kTile) * p.index_bytes;
        uint64_t id = 0;
        switch (p.index_bytes) {
            case 1: id = *id_address; break;
            case 2: id = *reinterpret_cast<const uint16_t*>(id_address); break;
            case 4: id = *reinterpret_cast<const uint32_t*>(id_address); break;
            default: id = *reinterpret_cast<const uint64_t*>(id_address); break;
        }
        const bool negative = p.index_signed && ((id >> (p.index_bytes * 8 - 1)) & 1u);
        if (negative || id >= p.vocabulary) {
            // Never form a table address from an invalid id
            // (standard_tiled_embedding.inl:167-172).
            if (threadIdx.x == 0 && chunk == 0) atomicOr(p.status, 1u);
            continue;
        }
        const uint32_t vector = chunk * kRowThreads + threadIdx.x;
        if (vector >= p.row.row_vectors) continue;
        const unsigned char* src = row_address(p.table, p.table.plane0, id, p.row.elem);
        unsigned char* dst = row_address(
                p.out, operand_plane(p.out, p.leading, index), r, p.row.elem);
        move_row_vectors(src, dst, p.row, vector);
    }
}

// ---- cache append --------------------------------------------------------------

struct AppendParams {
    Operand src;
    Operand dst;
    Leading leading;
    RowGeometry row;
    uint32_t rows;              // R: appended rows per plane
    uint64_t dst_rows;          // C: cache length
    uint64_t a;                 // scalar offset (positions == nullptr)
    const uint32_t* positions;  // per index of the first leading axis, or nullptr
    uint64_t planes_per_batch;  // logical planes per index of the first leading axis
    uint64_t total_rows;        // planes * R
    uint32_t chunks;
    uint32_t* status;           // batched only
};

__global__ void __launch_bounds__(kRowThreads)
cache_append_kernel(const AppendParams p) {
    const uint64_t items = p.total_rows * p.chunks;
    for (uint64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t chunk = static_cast<uint32_t>(item % p.chunks);
        const uint64_t global_row = item / p.chunks;
        const uint32_t r = static_cast<uint32_t>(global_row % p.rows);
        const uint64_t index = global_row / p.rows;
        uint64_t a = p.a;
        if (p.positions != nullptr) {
            a = p.positions[index / p.planes_per_batch];
            if (a > p.dst_rows || p.rows > p.dst_rows - a) {
                if (threadIdx.x == 0 && chunk == 0 && r == 0) atomicOr(p.status, 1u);
                continue;
            }
        }
        const uint32_t vector = chunk * kRowThreads + threadIdx.x;
        if (vector >= p.row.row_vectors) continue;
        const unsigned char* src = row_address(
                p.src, operand_plane(p.src, p.leading, index), r, p.row.elem);
        unsigned char* dst = row_address(
                p.dst, operand_plane(p.dst, p.leading, index), a + r, p.row.elem);
        move_row_vectors(src, dst, p.row, vector);
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
    if (fs.bytes == 0) {
        return fail(IOMB_ERR_UNSUPPORTED, "cache_append: sub-byte leaves are not implemented");
    }
    if (fs.rows > 0xFFFFFFFFull || fs.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "cache_append: matrix extent exceeds the kernel limit");
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
    p.total_rows = fs.planes * fs.rows;
    p.chunks = (p.row.row_vectors + kRowThreads - 1) / kRowThreads;
    p.status = status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (positions != nullptr) {
        if (cudaMemsetAsync(status, 0, sizeof(uint32_t), s) != cudaSuccess) {
            return check_launch("cache_append status reset");
        }
    }
    const unsigned grid = grid_for(p.total_rows * p.chunks, 16);
    cache_append_kernel<<<grid, kRowThreads, 0, s>>>(p);
    return check_launch("cache_append launch");
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
        case IOMB_I8: case IOMB_I16: case IOMB_I32: case IOMB_I64: index_signed = true; break;
        case IOMB_U8: case IOMB_U16: case IOMB_U32: case IOMB_U64: break;
        case IOMB_I2: case IOMB_U2: case IOMB_I4: case IOMB_U4:
            return fail(IOMB_ERR_UNSUPPORTED, "embedding: sub-byte index leaves are not implemented");
        default:
            return fail(IOMB_ERR_UNSUPPORTED, "embedding: index leaf is not integral");
    }
    if (ft.bytes == 0) {
        return fail(IOMB_ERR_UNSUPPORTED, "embedding: sub-byte payload leaves are not implemented");
    }
    if (fo.rows > 0xFFFFFFFFull || fo.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "embedding: matrix extent exceeds the kernel limit");
    }
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
    p.row = row_geometry(ft);
    p.run = static_cast<uint32_t>(fo.rows);
    p.index_bytes = fi.bytes;
    p.index_signed = index_signed ? 1u : 0u;
    p.vocabulary = ft.rows;
    p.total_rows = p.leading.planes * fo.rows;
    p.chunks = (p.row.row_vectors + kRowThreads - 1) / kRowThreads;
    p.status = status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Reset in queue order, as the reference does before its kernel
    // (src/shared/gpu_queue_operations.inl:899-914).
    if (cudaMemsetAsync(status, 0, sizeof(uint32_t), s) != cudaSuccess) {
        return check_launch("embedding status reset");
    }
    const unsigned grid = grid_for(p.total_rows * p.chunks, 16);
    embedding_kernel<<<grid, kRowThreads, 0, s>>>(p);
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
