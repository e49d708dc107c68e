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
#include "host.hpp"

namespace iomb {

constexpr int kRmsThreads = 256;
constexpr uint32_t kUnitCapBytes = 64 * 1024;

struct RmsParams {
    Operand x;
    Operand residual;   // fused only
    Operand sum;        // fused only
    Operand out;
    const unsigned char* scale_row;   // first tile of the [1,F] scale plane
    Leading leading;
    uint32_t rows;
    uint32_t cols;
    uint32_t tile_rows;
    uint32_t tile_cols;
    uint32_t group_rows;        // g
    uint32_t groups_per_band;   // 16 / g
    uint64_t units;
    float eps;
    uint32_t order;
};

__device__ __forceinline__ void cp_async_16(void* shared_dst, const void* global_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(global_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

template <int ELEM>
__device__ __forceinline__ float decode_element(const unsigned char* bytes) {
    if constexpr (ELEM == 2) {
        return __uint_as_float(
                static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(bytes)) << 16);
    } else {
        return *reinterpret_cast<const float*>(bytes);
    }
}

// sum + x*x with both operations rounded (never contracted).
__device__ __forceinline__ float accumulate_square(float sum, float value) {
    return __fadd_rn(sum, __fmul_rn(value, value));
}

template <int ELEM>
__device__ __forceinline__ uint4 add_vectors(uint4 a, uint4 b) {
    if constexpr (ELEM == 2) {
        auto word = [](uint32_t p, uint32_t q) {
            return pack_bf16x2_canonical(__fadd_rn(bf16_lo(p), bf16_lo(q)),
                                         __fadd_rn(bf16_hi(p), bf16_hi(q)));
        };
        return make_uint4(word(a.x, b.x), word(a.y, b.y), word(a.z, b.z), word(a.w, b.w));
    } else {
        auto word = [](uint32_t p, uint32_t q) {
            return f32_canonical_bits(__fadd_rn(__uint_as_float(p), __uint_as_float(q)));
        };
        return make_uint4(word(a.x, b.x), word(a.y, b.y), word(a.z, b.z), word(a.w, b.w));
    }
}

// Normalises one 16-byte vector: x from shared memory, w raw from shared memory.
template <int ELEM>
__device__ __forceinline__ uint4 normalize_vector(uint4 x, const unsigned char* w, float inv) {
    if constexpr (ELEM == 2) {
        const uint4 s = *reinterpret_cast<const uint4*>(w);
        auto word = [inv](uint32_t xv, uint32_t sv) {
            const float lo = __fmul_rn(__fmul_rn(bf16_lo(xv), inv), bf16_lo(sv));
            const float hi = __fmul_rn(__fmul_rn(bf16_hi(xv), inv), bf16_hi(sv));
            return pack_bf16x2_canonical(lo, hi);
        };
        return make_uint4(word(x.x, s.x), word(x.y, s.y), word(x.z, s.z), word(x.w, s.w));
    } else {
        const uint4 s = *reinterpret_cast<const uint4*>(w);
        auto word = [inv](uint32_t xv, uint32_t sv) {
            return f32_canonical_bits(
                    __fmul_rn(__fmul_rn(__uint_as_float(xv), inv), __uint_as_float(sv)));
        };
        return make_uint4(word(x.x, s.x), word(x.y, s.y), word(x.z, s.z), word(x.w, s.w));
    }
}

template <int ELEM>
__device__ __forceinline__ void store_vector_masked(
        unsigned char* address, uint4 value, uint32_t valid) {
    constexpr uint32_t kPerVector = 16 / ELEM;
    if (valid >= kPerVector) {
        store_u4_stream(address, value);
        return;
    }
    const uint32_t words[4] = {value.x, value.y, value.z, value.w};
    for (uint32_t e = 0; e < valid; ++e) {
        if constexpr (ELEM == 4) {
            reinterpret_cast<uint32_t*>(address)[e] = words[e];
        } else {
            reinterpret_cast<uint16_t*>(address)[e] =
                    static_cast<uint16_t>(words[e / 2] >> ((e & 1u) * 16));
        }
    }
}

// Shared memory: [unit: tile_cols * g * 16 * ELEM bytes][scale: tile_cols*16*ELEM]
//                [lanes: 16 rows x 16 floats][inverse: 16 floats]
template <int ELEM, bool FUSED>
__global__ void __launch_bounds__(kRmsThreads)
rmsnorm_kernel(const RmsParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kRowBytes = kTile * ELEM;          // one in-tile row
    constexpr uint32_t kVectorsPerRow = kRowBytes / 16;   // 2 (16-bit) or 4 (32-bit)
    constexpr uint32_t kPerVector = 16 / ELEM;
    const uint32_t g = p.group_rows;
    const uint32_t piece_bytes = g * kRowBytes;           // per tile
    const uint32_t piece_vectors = g * kVectorsPerRow;
    const uint32_t unit_vectors = p.tile_cols * piece_vectors;
    unsigned char* unit = smem;
    unsigned char* scale = unit + static_cast<size_t>(p.tile_cols) * piece_bytes;
    float* lanes = reinterpret_cast<float*>(scale + static_cast<size_t>(p.tile_cols) * kRowBytes);
    float* inverse = lanes + kTile * kTile;
    const uint32_t tid = threadIdx.x;

    // Stage row 0 of every scale tile once per CTA.
    for (uint32_t i = tid; i < p.tile_cols * kVectorsPerRow; i += kRmsThreads) {
        const uint32_t tile = i / kVectorsPerRow, v = i % kVectorsPerRow;
        cp_async_16(scale + i * 16, p.scale_row + static_cast<size_t>(tile) * kTileBytes + v * 16);
    }

    for (uint64_t u = blockIdx.x; u < p.units; u += gridDim.x) {
        const uint32_t group = static_cast<uint32_t>(u % p.groups_per_band);
        const uint64_t band = u / p.groups_per_band;
        const uint32_t tr = static_cast<uint32_t>(band % p.tile_rows);
        const uint64_t index = band / p.tile_rows;
        const uint32_t row0 = group * g;                         // first in-tile row
        const uint32_t rows_in_band = min(kTile, p.rows - tr * kTile);
        if (row0 >= rows_in_band) continue;                      // uniform per CTA
        const uint32_t live_rows = min(g, rows_in_band - row0);
        const size_t band_offset_rows = static_cast<size_t>(row0) * kRowBytes;
        auto band_base = [&](const Operand& operand) {
            const uint64_t plane = operand_plane(operand, p.leading, index);
            return operand.base
                    + (plane * operand.tile_rows + tr) * operand.tile_cols
                            * static_cast<uint64_t>(kTileBytes)
                    + band_offset_rows;
        };
        const unsigned char* x_band = band_base(p.x);
        unsigned char* out_band = band_base(p.out);

        // ---- stage the unit ---------------------------------------------
        if constexpr (!FUSED) {
            for (uint32_t i = tid; i < unit_vectors; i += kRmsThreads) {
                const uint32_t tile = i / piece_vectors, v = i % piece_vectors;
                cp_async_16(unit + static_cast<size_t>(i) * 16,
                            x_band + static_cast<size_t>(tile) * kTileBytes + v * 16);
            }
        } else {
            const unsigned char* r_band = band_base(p.residual);
            unsigned char* s_band = band_base(p.sum);
            constexpr uint32_t kBatch = 4;
            for (uint32_t i0 = tid; i0 < unit_vectors; i0 += kRmsThreads * kBatch) {
                uint4 a[kBatch], b[kBatch];
#pragma unroll
                for (uint32_t k = 0; k < kBatch; ++k) {
                    const uint32_t i = i0 + k * kRmsThreads;
                    if (i < unit_vectors) {
                        const uint32_t tile = i / piece_vectors, v = i % piece_vectors;
                        const size_t offset = static_cast<size_t>(tile) * kTileBytes + v * 16;
                        a[k] = load_u4_stream(x_band + offset);
                        b[k] = load_u4_stream(r_band + offset);
                    }
                }
#pragma unroll
                for (uint32_t k = 0; k < kBatch; ++k) {
                    const uint32_t i = i0 + k * kRmsThreads;
                    if (i < unit_vectors) {
                        const uint32_t tile = i / piece_vectors, v = i % piece_vectors;
                        const uint32_t row = v / kVectorsPerRow;
                        const uint32_t col = tile * kTile + (v % kVectorsPerRow) * kPerVector;
                        const uint4 s = add_vectors<ELEM>(a[k], b[k]);
                        *reinterpret_cast<uint4*>(unit + static_cast<size_t>(i) * 16) = s;
                        if (row < live_rows && col < p.cols) {
                            store_vector_masked<ELEM>(
                                    s_band + static_cast<size_t>(tile) * kTileBytes + v * 16, s,
                                    min(kPerVector, p.cols - col));
                        }
                    }
                }
            }
        }
        cp_async_wait_all();
        __syncthreads();

        // ---- pass 1: row sums of squares ---------------------------------
        if (p.order == IOMB_RMS_LANES16) {
            if (tid < g * kTile) {
                const uint32_t row = tid / kTile, lane = tid % kTile;
                const unsigned char* cursor = unit + (row * kTile + lane) * ELEM;
                const uint32_t full_tiles = p.cols / kTile;
                float acc = 0.0f;
#pragma unroll 8
                for (uint32_t tile = 0; tile < full_tiles; ++tile) {
                    acc = accumulate_square(acc, decode_element<ELEM>(cursor));
                    cursor += piece_bytes;
                }
                if (full_tiles < p.tile_cols && lane < p.cols % kTile) {
                    acc = accumulate_square(acc, decode_element<ELEM>(cursor));
                }
                lanes[row * kTile + lane] = acc;
            }
            __syncthreads();
            if (tid < g) {
                const float* l = lanes + tid * kTile;
                float total[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    total[j] = __fadd_rn(__fadd_rn(__fadd_rn(l[j], l[j + 4]), l[j + 8]), l[j + 12]);
                }
                const float sum = __fadd_rn(__fadd_rn(total[0], total[2]),
                                            __fadd_rn(total[1], total[3]));
                const float mean = __fdiv_rn(sum, static_cast<float>(p.cols));
                const float root = __fsqrt_rn(__fadd_rn(mean, p.eps));
                inverse[tid] = __fdiv_rn(1.0f, root);
            }
        } else {
            if (tid < g) {
                const unsigned char* cursor = unit + tid * kRowBytes;
                float sum = 0.0f;
                uint32_t remaining = p.cols;
                for (uint32_t tile = 0; tile < p.tile_cols; ++tile) {
                    const uint32_t count = min(kTile, remaining);
                    if (count == kTile) {
#pragma unroll
                        for (uint32_t c = 0; c < kTile; ++c) {
                            sum = accumulate_square(sum, decode_element<ELEM>(cursor + c * ELEM));
                        }
                    } else {
                        for (uint32_t c = 0; c < count; ++c) {
                            sum = accumulate_square(sum, decode_element<ELEM>(cursor + c * ELEM));
                        }
                    }
                    remaining -= count;
                    cursor += piece_bytes;
                }
                const float mean = __fdiv_rn(sum, static_cast<float>(p.cols));
                const float root = __fsqrt_rn(__fadd_rn(mean, p.eps));
                inverse[tid] = __fdiv_rn(1.0f, root);
            }
        }
        __syncthreads();

        // ---- pass 2: normalise, scale, encode, store ----------------------
        for (uint32_t i = tid; i < unit_vectors; i += kRmsThreads) {
            const uint32_t tile = i / piece_vectors, v = i % piece_vectors;
            const uint32_t row = v / kVectorsPerRow;
            const uint32_t cv = v % kVectorsPerRow;
            const uint32_t col = tile * kTile + cv * kPerVector;
            if (row >= live_rows || col >= p.cols) continue;
            const uint4 xv = *reinterpret_cast<const uint4*>(unit + static_cast<size_t>(i) * 16);
            const uint4 y = normalize_vector<ELEM>(
                    xv, scale + (static_cast<size_t>(tile) * kVectorsPerRow + cv) * 16,
                    inverse[row]);
            store_vector_masked<ELEM>(
                    out_band + static_cast<size_t>(tile) * kTileBytes + v * 16, y,
                    min(kPerVector, p.cols - col));
        }
        __syncthreads();   // the unit buffer is reused by the next iteration
    }
    cp_async_wait_all();
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
    uint32_t g = kTile;
    while (g > 1 && g * row_bytes > kUnitCapBytes) g /= 2;
    const uint64_t smem_bytes = g * row_bytes + row_bytes + (kTile * kTile + kTile) * sizeof(float);
    if (smem_bytes > 200 * 1024) {
        return fail(IOMB_ERR_UNSUPPORTED, "rmsnorm: feature extent exceeds the staging capacity");
    }

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
    p.group_rows = g;
    p.groups_per_band = kTile / g;
    p.units = p.leading.planes * p.tile_rows * p.groups_per_band;
    p.eps = eps;
    p.order = static_cast<uint32_t>(order);

    auto kernel = elem == 2 ? (fused ? rmsnorm_kernel<2, true> : rmsnorm_kernel<2, false>)
                            : (fused ? rmsnorm_kernel<4, true> : rmsnorm_kernel<4, false>);
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem_bytes)) != cudaSuccess) {
        return check_launch("rmsnorm shared-memory attribute");
    }
    const unsigned per_sm = static_cast<unsigned>(
            smem_bytes + 1024 > 0 ? (227 * 1024) / (smem_bytes + 1024) : 1);
    const unsigned grid = grid_for(p.units, per_sm > 0 ? (per_sm > 8 ? 8 : per_sm) : 1);
    kernel<<<grid, kRmsThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(p);
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
