// Host-side admission helpers and the layout entry points that need no device.
#include "host.hpp"

#include <stdio.h>
#include <string.h>

#include <mutex>
#include <set>
#include <utility>

namespace iomb {

namespace {
thread_local char g_error[256] = "";
thread_local char g_launch[160] = "";
}  // namespace

void note_launch(const char* text) {
    snprintf(g_launch, sizeof g_launch, "%s", text ? text : "");
}

void set_error(const char* text) {
    snprintf(g_error, sizeof g_error, "%s", text ? text : "");
}

int fail(int status, const char* text) {
    set_error(text);
    return status;
}

int check_launch(const char* what) {
    const cudaError_t error = cudaGetLastError();
    if (error != cudaSuccess) {
        char text[256];
        snprintf(text, sizeof text, "%s: %s", what, cudaGetErrorString(error));
        return fail(IOMB_ERR_DEVICE, text);
    }
    return IOMB_OK;
}

int sm_count() {
    static int cached[64];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        cudaGetLastError();
        return 0;
    }
    if (cached[device] == 0) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device)
                != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        cached[device] = count;
    }
    return cached[device];
}

int allow_full_shared_memory(const void* kernel) {
    static std::mutex guard;
    static std::set<std::pair<const void*, int>> prepared;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return check_launch("current device");
    const std::lock_guard<std::mutex> lock(guard);
    if (prepared.count({kernel, device}) != 0) return IOMB_OK;
    // Static and dynamic shared memory share the 227 KiB.
    cudaFuncAttributes facts{};
    if (cudaFuncGetAttributes(&facts, kernel) != cudaSuccess) {
        return check_launch("kernel attributes");
    }
    const int dynamic = 227 * 1024 - static_cast<int>(facts.sharedSizeBytes);
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic)
            != cudaSuccess) {
        return check_launch("shared-memory attribute");
    }
    prepared.insert({kernel, device});
    return IOMB_OK;
}

unsigned grid_for(uint64_t work_items, unsigned ctas_per_sm) {
    const int sms = sm_count();
    uint64_t grid = static_cast<uint64_t>(sms > 0 ? sms : 148) * ctas_per_sm;
    if (grid > work_items) grid = work_items;
    if (grid == 0) grid = 1;
    return static_cast<unsigned>(grid);
}

unsigned grid_one_shot(uint64_t work_items) {
    if (work_items == 0) return 1;
    return static_cast<unsigned>(work_items > 0x7FFFFFFFull ? 0x7FFFFFFFull : work_items);
}

static bool mul_overflows(uint64_t a, uint64_t b, uint64_t* out) {
    return __builtin_mul_overflow(a, b, out);
}
static bool add_overflows(uint64_t a, uint64_t b, uint64_t* out) {
    return __builtin_add_overflow(a, b, out);
}

int check_view(const iomb_view* view, const char* what, ViewFacts* facts) {
    char text[200];
    if (view == nullptr) {
        snprintf(text, sizeof text, "%s: view is null", what);
        return fail(IOMB_ERR_INVALID_ARGUMENT, text);
    }
    const uint32_t bits = iomb_dtype_bits(view->dtype);
    if (bits == 0) {
        snprintf(text, sizeof text, "%s: unknown DataType value", what);
        return fail(IOMB_ERR_INVALID_ARGUMENT, text);
    }
    if (view->rank < 2 || view->rank > IOMB_MAX_RANK) {
        snprintf(text, sizeof text, "%s: requires rank two through eight", what);
        return fail(IOMB_ERR_INVALID_ARGUMENT, text);
    }
    for (uint32_t i = 0; i < view->rank; ++i) {
        if (view->dims[i] == 0) {
            snprintf(text, sizeof text, "%s: dimensions must be nonzero", what);
            return fail(IOMB_ERR_INVALID_ARGUMENT, text);
        }
    }
    if (view->base == nullptr) {
        snprintf(text, sizeof text, "%s: view has no stable owner handle", what);
        return fail(IOMB_ERR_INVALID_ARGUMENT, text);
    }
    if (reinterpret_cast<uintptr_t>(view->base) % 32 != 0) {
        snprintf(text, sizeof text, "%s: owner storage is not 32-byte aligned", what);
        return fail(IOMB_ERR_INVALID_ARGUMENT, text);
    }
    ViewFacts f{};
    f.bits = bits;
    f.bytes = bits % 8 == 0 ? bits / 8 : 0;
    f.leading = view->rank - 2;
    f.rows = view->dims[view->rank - 2];
    f.cols = view->dims[view->rank - 1];
    uint64_t padded_rows = 0, padded_cols = 0;
    if (add_overflows(f.rows, kTile - 1, &padded_rows)
            || add_overflows(f.cols, kTile - 1, &padded_cols)) {
        snprintf(text, sizeof text, "%s: tile count overflows", what);
        return fail(IOMB_ERR_OVERFLOW, text);
    }
    f.tile_rows = padded_rows / kTile;
    f.tile_cols = padded_cols / kTile;
    uint64_t tiles = 0, plane_bits = 0;
    if (mul_overflows(f.tile_rows, f.tile_cols, &tiles)
            || mul_overflows(tiles, static_cast<uint64_t>(kTileSlots) * bits, &plane_bits)) {
        snprintf(text, sizeof text, "%s: plane size overflows", what);
        return fail(IOMB_ERR_OVERFLOW, text);
    }
    f.plane_bytes = plane_bits / 8;  // 256 slots * bits is always a whole byte count
    f.planes = 1;
    f.max_plane = view->plane_offset;
    for (uint32_t i = 0; i < f.leading; ++i) {
        if (view->plane_strides[i] == 0) {
            snprintf(text, sizeof text, "%s: view does not permit zero plane strides", what);
            return fail(IOMB_ERR_INVALID_ARGUMENT, text);
        }
        uint64_t span = 0;
        if (mul_overflows(f.planes, view->dims[i], &f.planes)
                || mul_overflows(view->dims[i] - 1, view->plane_strides[i], &span)
                || add_overflows(f.max_plane, span, &f.max_plane)) {
            snprintf(text, sizeof text, "%s: plane address overflows", what);
            return fail(IOMB_ERR_OVERFLOW, text);
        }
    }
    uint64_t end_plane = 0, end_bytes = 0;
    if (add_overflows(f.max_plane, 1, &end_plane)
            || mul_overflows(end_plane, f.plane_bytes, &end_bytes)) {
        snprintf(text, sizeof text, "%s: view size overflows", what);
        return fail(IOMB_ERR_OVERFLOW, text);
    }
    if (end_bytes > view->storage_bytes) {
        snprintf(text, sizeof text, "%s: view exceeds its owner storage", what);
        return fail(IOMB_ERR_INVALID_ARGUMENT, text);
    }
    if (f.tile_rows > 0xFFFFFFFFull || f.tile_cols > 0xFFFFFFFFull) {
        snprintf(text, sizeof text, "%s: matrix extent exceeds the kernel limit", what);
        return fail(IOMB_ERR_UNSUPPORTED, text);
    }
    *facts = f;
    return IOMB_OK;
}

bool same_window(const iomb_view& a, const iomb_view& b) {
    if (a.base != b.base || a.dtype != b.dtype || a.rank != b.rank
            || a.plane_offset != b.plane_offset) {
        return false;
    }
    for (uint32_t i = 0; i < a.rank; ++i) {
        if (a.dims[i] != b.dims[i]) return false;
    }
    for (uint32_t i = 0; i + 2 < a.rank; ++i) {
        if (a.plane_strides[i] != b.plane_strides[i]) return false;
    }
    return true;
}

bool storage_overlaps(const iomb_view& a, const ViewFacts& fa,
                      const iomb_view& b, const ViewFacts& fb) {
    const uintptr_t a_begin =
            reinterpret_cast<uintptr_t>(a.base) + a.plane_offset * fa.plane_bytes;
    const uintptr_t a_end =
            reinterpret_cast<uintptr_t>(a.base) + (fa.max_plane + 1) * fa.plane_bytes;
    const uintptr_t b_begin =
            reinterpret_cast<uintptr_t>(b.base) + b.plane_offset * fb.plane_bytes;
    const uintptr_t b_end =
            reinterpret_cast<uintptr_t>(b.base) + (fb.max_plane + 1) * fb.plane_bytes;
    return a_begin < b_end && b_begin < a_end;
}

void collapse_leading(uint32_t lead_rank, const uint64_t* result_dims,
                      uint64_t strides[][kMaxLead], uint32_t count,
                      Leading* leading) {
    uint64_t dims[kMaxLead];
    uint32_t n = 0;
    // Drop unit axes.
    for (uint32_t axis = 0; axis < lead_rank; ++axis) {
        if (result_dims[axis] == 1) continue;
        dims[n] = result_dims[axis];
        for (uint32_t k = 0; k < count; ++k) strides[k][n] = strides[k][axis];
        ++n;
    }
    // Merge an outer axis into the next inner one when every operand steps
    // through them as one dense run.
    uint32_t write = 0;
    for (uint32_t axis = 0; axis < n; ++axis) {
        if (write > 0) {
            bool mergeable = true;
            for (uint32_t k = 0; k < count && mergeable; ++k) {
                uint64_t span = 0;
                if (mul_overflows(strides[k][axis], dims[axis], &span)
                        || strides[k][write - 1] != span) {
                    mergeable = false;
                }
            }
            if (mergeable) {
                dims[write - 1] *= dims[axis];
                for (uint32_t k = 0; k < count; ++k) {
                    strides[k][write - 1] = strides[k][axis];
                }
                continue;
            }
        }
        dims[write] = dims[axis];
        for (uint32_t k = 0; k < count; ++k) strides[k][write] = strides[k][axis];
        ++write;
    }
    leading->count = write;
    leading->planes = 1;
    for (uint32_t axis = 0; axis < kMaxLead; ++axis) {
        leading->dims[axis] = axis < write ? dims[axis] : 1;
        if (axis < write) leading->planes *= dims[axis];
        for (uint32_t k = 0; k < count; ++k) {
            if (axis >= write) strides[k][axis] = 0;
        }
    }
    bool contiguous = write <= 1;
    if (write == 1) {
        for (uint32_t k = 0; k < count; ++k) {
            if (strides[k][0] != 1) contiguous = false;
        }
    }
    leading->contiguous = contiguous ? 1u : 0u;
}

Operand make_operand(const iomb_view& view, const ViewFacts& facts,
                     const uint64_t* aligned_strides, const Leading& leading,
                     bool bc_rows, bool bc_cols) {
    Operand operand{};
    operand.base = static_cast<unsigned char*>(view.base);
    operand.plane0 = view.plane_offset;
    for (uint32_t axis = 0; axis < kMaxLead; ++axis) {
        operand.stride[axis] = axis < leading.count ? aligned_strides[axis] : 0;
    }
    operand.tile_rows = static_cast<uint32_t>(facts.tile_rows);
    operand.tile_cols = static_cast<uint32_t>(facts.tile_cols);
    operand.bc_rows = bc_rows ? 1u : 0u;
    operand.bc_cols = bc_cols ? 1u : 0u;
    return operand;
}

}  // namespace iomb

extern "C" {

const char* iomb_last_error(void) { return iomb::g_error; }

const char* iomb_last_launch(void) { return iomb::g_launch; }

uint32_t iomb_abi_version(void) { return 2; }

int iomb_prepare_device(void* stream) {
    if (iomb::sm_count() <= 0) return iomb::fail(IOMB_ERR_DEVICE, "no CUDA device is current");
    int status = iomb::prepare_rmsnorm_kernels();
    if (status == IOMB_OK) status = iomb::prepare_rmsnorm_long_kernels();
    if (status == IOMB_OK) status = iomb::prepare_sdpa_kernels();
    if (status == IOMB_OK) status = iomb::prepare_silu(static_cast<cudaStream_t>(stream));
    return status;
}

uint32_t iomb_dtype_bits(uint32_t dtype) {
    switch (dtype) {
        case IOMB_BOOL: return 8;
        case IOMB_I2: case IOMB_U2: return 2;
        case IOMB_I4: case IOMB_U4: case IOMB_F4_E2M1: return 4;
        case IOMB_F6_E2M3: case IOMB_F6_E3M2: return 6;
        case IOMB_I8: case IOMB_U8: case IOMB_F8_E4M3FN: case IOMB_F8_E5M2:
        case IOMB_F8_E8M0: return 8;
        case IOMB_I16: case IOMB_U16: case IOMB_F16: case IOMB_BF16: return 16;
        case IOMB_I32: case IOMB_U32: case IOMB_F32: return 32;
        case IOMB_I64: case IOMB_U64: case IOMB_F64: return 64;
        default: return 0;
    }
}

static int shape_elements(const uint64_t* dims, uint32_t rank, bool padded,
                          uint64_t* elements) {
    if (dims == nullptr || rank < 2 || rank > IOMB_MAX_RANK) {
        return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "shape requires rank two through eight");
    }
    uint64_t count = 1;
    for (uint32_t i = 0; i < rank; ++i) {
        uint64_t extent = dims[i];
        if (extent == 0) {
            return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "tensor dimensions must be nonzero");
        }
        if (padded && i + 2 >= rank) {
            if (__builtin_add_overflow(extent, iomb::kTile - 1, &extent)) {
                return iomb::fail(IOMB_ERR_OVERFLOW, "padded dimension overflows");
            }
            extent = extent / iomb::kTile * iomb::kTile;
        }
        if (__builtin_mul_overflow(count, extent, &count)) {
            return iomb::fail(IOMB_ERR_OVERFLOW, "tensor element count overflows");
        }
    }
    *elements = count;
    return IOMB_OK;
}

static int shape_bytes(const uint64_t* dims, uint32_t rank, uint32_t dtype,
                       bool padded, uint64_t* out_bytes) {
    const uint32_t bits = iomb_dtype_bits(dtype);
    if (bits == 0) return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "unknown DataType value");
    if (out_bytes == nullptr) return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "null result");
    uint64_t elements = 0;
    const int status = shape_elements(dims, rank, padded, &elements);
    if (status != IOMB_OK) return status;
    uint64_t total_bits = 0;
    if (__builtin_mul_overflow(elements, static_cast<uint64_t>(bits), &total_bits)
            || total_bits > UINT64_MAX - 7) {
        return iomb::fail(IOMB_ERR_OVERFLOW, "byte count overflows");
    }
    *out_bytes = (total_bits + 7) / 8;
    return IOMB_OK;
}

int iomb_tiled_storage_nbytes(const uint64_t* dims, uint32_t rank, uint32_t dtype,
                              uint64_t* out_bytes) {
    return shape_bytes(dims, rank, dtype, true, out_bytes);
}

int iomb_logical_nbytes(const uint64_t* dims, uint32_t rank, uint32_t dtype,
                        uint64_t* out_bytes) {
    return shape_bytes(dims, rank, dtype, false, out_bytes);
}

uint64_t iomb_plane_slot(uint64_t rows, uint64_t columns, uint64_t plane,
                         uint64_t row, uint64_t column) {
    const uint64_t tile_rows = (rows + iomb::kTile - 1) / iomb::kTile;
    const uint64_t tile_columns = (columns + iomb::kTile - 1) / iomb::kTile;
    const uint64_t tile = plane * tile_rows * tile_columns
            + (row / iomb::kTile) * tile_columns + column / iomb::kTile;
    return tile * iomb::kTileSlots + (row % iomb::kTile) * iomb::kTile
            + column % iomb::kTile;
}

}  // extern "C"
