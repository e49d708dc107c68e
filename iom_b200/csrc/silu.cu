// SiLU (x * sigmoid(x)) and SiLU followed by the gate multiply on tiled storage.
//
// Replaces GpuQueue::silu_impl + silu_kernel of the reference
// (src/cuda/copy.cu:452-571), which evaluates scalar_silu
// (src/shared/scalar_silu.hpp:66-101) on an FP64 carrier one 16-feature packet
// per thread. The arithmetic kept here is exactly that: decode the leaf,
// evaluate on FP64 (x / (1 + exp(-x)) for x >= 0, ((x*t)*t) / (1 + t*t) with
// t = exp(x/2) below zero, every operation rounded separately), one RNE encode.
//
// BF16 has 65 536 codes, so the whole function is a table: it is built once per
// device by silu_table_kernel with the FP64 evaluator and lives in a 128 KiB
// array inside this library. (For BF16 the FP64 carrier and the FP32 carrier of
// the reference CPU backend give the same code for every input; the parity
// tests check all 65 536.) Large dense requests stage the table in shared
// memory (one persistent CTA per SM) and turn every element into one
// shared-memory load; small or ragged requests read it through L1/L2. The F32
// leaf evaluates on FP64 per element.
//
// iomb_silu_mul fuses the multiply that follows SiLU in the decoder MLP
// (src/session.cpp:2020-2030): out = silu(x) * up with the activated value
// rounded to the leaf first (and stored when the caller passes a view for it),
// so the result equals iomb_silu followed by iomb_binary(MUL) bit for bit.
#include "host.hpp"

#include <mutex>

namespace iomb {

// ---- FP64 evaluation and encoders ------------------------------------------

// scalar_silu_detail::evaluate (src/shared/scalar_silu.hpp:70-89) on FP64.
__device__ __forceinline__ double silu_evaluate(double x) {
    if (x != x) return __longlong_as_double(0x7FF8000000000000ll);
    if (fabs(x) == __longlong_as_double(0x7FF0000000000000ll)) {
        return x < 0.0 ? -0.0 : x;
    }
    if (x == 0.0) return x;
    if (x >= 0.0) {
        return __ddiv_rn(x, __dadd_rn(1.0, exp(-x)));
    }
    const double t = exp(__dmul_rn(x, 0.5));
    const double numerator = __dmul_rn(__dmul_rn(x, t), t);
    return __ddiv_rn(numerator, __dadd_rn(1.0, __dmul_rn(t, t)));
}

// One round-to-nearest-even from FP64 straight to BF16 (never through FP32),
// subnormal results included; every NaN becomes the positive quiet NaN.
__device__ __forceinline__ uint32_t f64_to_bf16(double value) {
    const uint64_t bits = static_cast<uint64_t>(__double_as_longlong(value));
    const uint32_t sign = static_cast<uint32_t>(bits >> 48) & 0x8000u;
    const uint64_t magnitude = bits & 0x7FFFFFFFFFFFFFFFull;
    if (magnitude > 0x7FF0000000000000ull) return 0x7FC0u;
    if (magnitude == 0x7FF0000000000000ull) return sign | 0x7F80u;
    const int exponent = static_cast<int>(magnitude >> 52) - 1023;
    if (exponent < -140) return sign;     // below a quarter of the smallest subnormal (and FP64 subnormals)
    const uint64_t significand = (magnitude & 0x000FFFFFFFFFFFFFull) | 0x0010000000000000ull;
    // Normal results keep 8 significant bits; below 2^-126 the quantum stays 2^-133.
    const int shift = 45 + (exponent < -126 ? -126 - exponent : 0);
    uint64_t quotient = significand >> shift;
    const uint64_t remainder = significand & ((1ull << shift) - 1ull);
    const uint64_t half = 1ull << (shift - 1);
    if (remainder > half || (remainder == half && (quotient & 1ull))) ++quotient;
    uint32_t code;
    if (exponent >= -126) {
        // quotient in [128, 256]; 256 carries into the exponent field by itself.
        code = (static_cast<uint32_t>(exponent + 127) << 7) + static_cast<uint32_t>(quotient - 128);
        if (code >= 0x7F80u) code = 0x7F80u;
    } else {
        code = static_cast<uint32_t>(quotient);   // 128 is the smallest normal, as it should be
    }
    return sign | code;
}

__device__ __forceinline__ double bf16_to_f64(uint32_t code) {
    return static_cast<double>(__uint_as_float(code << 16));
}

// F32 leaf: decode, evaluate, one RNE encode, canonical NaN.
__device__ __forceinline__ uint32_t silu_f32_bits(uint32_t raw) {
    const float result = __double2float_rn(silu_evaluate(static_cast<double>(__uint_as_float(raw))));
    return f32_canonical_bits(result);
}

// ---- the BF16 table ---------------------------------------------------------

__device__ __align__(16) uint16_t g_silu_bf16[65536];

__global__ void silu_table_kernel() {
    const uint32_t code = blockIdx.x * blockDim.x + threadIdx.x;
    if (code < 65536u) {
        g_silu_bf16[code] = static_cast<uint16_t>(f64_to_bf16(silu_evaluate(bf16_to_f64(code))));
    }
}

// Builds the table the first time a device is used (launch on the caller's
// stream, then one wait for it: the only synchronisation this file ever does) and
// returns its device address.
static int silu_table(cudaStream_t stream, const uint16_t** table) {
    constexpr int kMaxDevices = 64;
    static std::mutex guard;
    static const uint16_t* tables[kMaxDevices] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        return fail(IOMB_ERR_DEVICE, "silu: cannot identify the current device");
    }
    std::lock_guard<std::mutex> lock(guard);
    if (tables[device] == nullptr) {
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, g_silu_bf16) != cudaSuccess) {
            return check_launch("silu table address");
        }
        silu_table_kernel<<<65536 / 256, 256, 0, stream>>>();
        if (cudaStreamSynchronize(stream) != cudaSuccess) {
            return fail(IOMB_ERR_DEVICE,
                        "silu: the first call on a device builds a table and must not be "
                        "made while the stream is being captured");
        }
        tables[device] = static_cast<const uint16_t*>(address);
    }
    *table = tables[device];
    return IOMB_OK;
}

// ---- per-vector work ---------------------------------------------------------

// Two BF16 codes of one word through the table (any 16-bit-addressable space).
template <typename Table>
__device__ __forceinline__ uint32_t silu_word_bf16(uint32_t word, Table table) {
    return static_cast<uint32_t>(table[word & 0xFFFFu])
            | (static_cast<uint32_t>(table[word >> 16]) << 16);
}

template <int ELEM, typename Table>
__device__ __forceinline__ uint4 silu_vector(uint4 x, Table table) {
    if constexpr (ELEM == 2) {
        return make_uint4(silu_word_bf16(x.x, table), silu_word_bf16(x.y, table),
                          silu_word_bf16(x.z, table), silu_word_bf16(x.w, table));
    } else {
        return make_uint4(silu_f32_bits(x.x), silu_f32_bits(x.y), silu_f32_bits(x.z),
                          silu_f32_bits(x.w));
    }
}

// activated * up, one IEEE binary32 product and one RNE encode, canonical NaN
// (the arithmetic of iomb_binary(MUL)).
template <int ELEM>
__device__ __forceinline__ uint4 gate_vector(uint4 activated, uint4 up) {
    if constexpr (ELEM == 2) {
        auto word = [](uint32_t a, uint32_t b) {
            return pack_bf16x2_canonical(__fmul_rn(bf16_lo(a), bf16_lo(b)),
                                         __fmul_rn(bf16_hi(a), bf16_hi(b)));
        };
        return make_uint4(word(activated.x, up.x), word(activated.y, up.y),
                          word(activated.z, up.z), word(activated.w, up.w));
    } else {
        auto word = [](uint32_t a, uint32_t b) {
            return f32_canonical_bits(__fmul_rn(__uint_as_float(a), __uint_as_float(b)));
        };
        return make_uint4(word(activated.x, up.x), word(activated.y, up.y),
                          word(activated.z, up.z), word(activated.w, up.w));
    }
}

// ---- dense streams -------------------------------------------------------------

constexpr int kSiluUnroll = 4;
constexpr int kSiluThreads = 256;
constexpr int kSiluStagedThreads = 1024;   // one CTA per SM next to the 128 KiB table
constexpr uint32_t kSiluTableBytes = 65536 * sizeof(uint16_t);

// Every operand is a dense run of whole tiles: the storages are walked as linear
// streams of 16-byte vectors, kSiluUnroll per thread in flight. STAGED (BF16,
// large requests): one persistent CTA per SM first copies the table into shared
// memory, so that every element costs one shared-memory load whatever the
// values are; otherwise one chunk per CTA in launch order and the table, if any,
// is read through L1. (Staging only the 15 exponents outside which the function
// has closed forms, 7.5 KiB, allowed several CTAs per SM but its index
// arithmetic made it 10 % slower.)
template <int ELEM, bool FUSED, bool STAGED>
__global__ void __launch_bounds__(STAGED ? kSiluStagedThreads : kSiluThreads)
silu_stream_kernel(const uint4* __restrict__ x, const uint4* __restrict__ up,
                   uint4* __restrict__ activated, uint4* __restrict__ out, uint64_t vectors,
                   const uint16_t* __restrict__ table) {
    extern __shared__ __align__(16) unsigned char staged_bytes[];
    constexpr int kThreads = STAGED ? kSiluStagedThreads : kSiluThreads;
    const uint16_t* lookup = table;
    if constexpr (STAGED) {
        uint4* staged = reinterpret_cast<uint4*>(staged_bytes);
        const uint4* source = reinterpret_cast<const uint4*>(table);
        for (uint32_t i = threadIdx.x; i < kSiluTableBytes / 16; i += kThreads) {
            staged[i] = __ldg(source + i);
        }
        __syncthreads();
        lookup = reinterpret_cast<const uint16_t*>(staged_bytes);
    }
    constexpr uint64_t kChunk = static_cast<uint64_t>(kThreads) * kSiluUnroll;
    const uint64_t chunks = (vectors + kChunk - 1) / kChunk;
    for (uint64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
        const uint64_t base = chunk * kChunk + threadIdx.x;
        uint4 xv[kSiluUnroll], uv[kSiluUnroll];
#pragma unroll
        for (int u = 0; u < kSiluUnroll; ++u) {
            const uint64_t index = base + static_cast<uint64_t>(u) * kThreads;
            if (index < vectors) {
                xv[u] = load_u4_stream(x + index);
                if constexpr (FUSED) uv[u] = load_u4_stream(up + index);
            }
        }
#pragma unroll
        for (int u = 0; u < kSiluUnroll; ++u) {
            const uint64_t index = base + static_cast<uint64_t>(u) * kThreads;
            if (index < vectors) {
                const uint4 value = silu_vector<ELEM>(xv[u], lookup);
                if constexpr (FUSED) {
                    if (activated != nullptr) store_u4_stream(activated + index, value);
                    store_u4_stream(out + index, gate_vector<ELEM>(value, uv[u]));
                } else {
                    store_u4_stream(out + index, value);
                }
            }
        }
    }
}

// ---- general case: one warp per tile, stores masked to the logical extents ------

struct SiluParams {
    Operand x;
    Operand up;          // fused only
    Operand activated;   // fused only, optional
    Operand out;
    Leading leading;
    uint32_t rows;
    uint32_t cols;
    uint32_t tile_rows;
    uint32_t tile_cols;
    uint32_t has_activated;
    uint64_t items;      // planes * tile_rows * tile_cols
    const uint16_t* table;
};

template <int ELEM>
__device__ __forceinline__ void silu_store_masked(unsigned char* address, uint4 value,
                                                  uint32_t valid) {
    constexpr uint32_t kPerVector = 16 / ELEM;
    if (valid >= kPerVector) {
        store_u4(address, value);
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

template <int ELEM, bool FUSED>
__global__ void __launch_bounds__(kSiluThreads)
silu_tiled_kernel(const SiluParams p) {
    constexpr uint32_t kTileBytes = kTileSlots * ELEM;
    constexpr uint32_t kTileVectors = kTileBytes / 16;
    constexpr uint32_t kPerVector = 16 / ELEM;
    constexpr int kWarps = kSiluThreads / 32;
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warp = static_cast<uint64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * kWarps;
    for (uint64_t item = warp; item < p.items; item += warps) {
        const uint32_t tc = static_cast<uint32_t>(item % p.tile_cols);
        const uint64_t band = item / p.tile_cols;
        const uint32_t tr = static_cast<uint32_t>(band % p.tile_rows);
        const uint64_t index = band / p.tile_rows;
        const uint64_t tile_in_plane = static_cast<uint64_t>(tr) * p.tile_cols + tc;
        auto tile_of = [&](const Operand& operand) {
            return operand.base
                    + (operand_plane(operand, p.leading, index) * p.tile_rows * p.tile_cols
                       + tile_in_plane) * kTileBytes;
        };
        const unsigned char* x_tile = tile_of(p.x);
        unsigned char* out_tile = tile_of(p.out);
        const uint32_t rows_left = p.rows - tr * kTile;
        const uint32_t cols_left = p.cols - tc * kTile;
        for (uint32_t k = lane; k < kTileVectors; k += 32) {
            const uint32_t slot = k * kPerVector;
            const uint32_t row = slot / kTile, col = slot % kTile;
            if (row >= rows_left || col >= cols_left) continue;
            const uint32_t valid = min(kPerVector, cols_left - col);
            const uint4 value = silu_vector<ELEM>(load_u4(x_tile + k * 16), p.table);
            if constexpr (FUSED) {
                if (p.has_activated) silu_store_masked<ELEM>(tile_of(p.activated) + k * 16, value, valid);
                silu_store_masked<ELEM>(out_tile + k * 16,
                                        gate_vector<ELEM>(value, load_u4(tile_of(p.up) + k * 16)),
                                        valid);
            } else {
                silu_store_masked<ELEM>(out_tile + k * 16, value, valid);
            }
        }
    }
}

// ---- admission and dispatch -----------------------------------------------------

static bool silu_same_shape(const iomb_view& a, const iomb_view& b) {
    if (a.rank != b.rank) return false;
    for (uint32_t i = 0; i < a.rank; ++i) {
        if (a.dims[i] != b.dims[i]) return false;
    }
    return true;
}

// Rules of validate_silu (src/device_ops_neural.cpp:391-434): equal shapes and
// specifications, the output shares neither an owner nor a byte with an input.
static int silu_dispatch(const iomb_view* x, const iomb_view* up, const iomb_view* activated,
                         const iomb_view* out, void* stream) {
    const bool fused = up != nullptr;
    const iomb_view* views[4] = {x, out, up, activated};
    const char* names[4] = {"silu x", "silu out", "silu_mul up", "silu_mul activated"};
    ViewFacts facts[4] = {};
    const uint32_t count = fused ? (activated != nullptr ? 4u : 3u) : 2u;
    for (uint32_t k = 0; k < count; ++k) {
        const int status = check_view(views[k], names[k], &facts[k]);
        if (status != IOMB_OK) return status;
    }
    for (uint32_t k = 1; k < count; ++k) {
        if (!silu_same_shape(*x, *views[k])) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "silu views must have identical shape");
        }
        if (views[k]->dtype != x->dtype) {
            return fail(IOMB_ERR_INVALID_ARGUMENT, "silu specifications must match");
        }
    }
    // Written views (out, activated) against every other view.
    for (uint32_t w = 1; w < count; w += 2) {
        for (uint32_t k = 0; k < count; ++k) {
            if (k == w) continue;
            if (views[w]->base == views[k]->base) {
                return fail(IOMB_ERR_INVALID_ARGUMENT, "silu output aliases another operand's owner");
            }
            if (storage_overlaps(*views[w], facts[w], *views[k], facts[k])) {
                return fail(IOMB_ERR_INVALID_ARGUMENT, "silu output storage range overlaps an operand");
            }
        }
    }
    if (x->dtype != IOMB_BF16 && x->dtype != IOMB_F32) {
        return fail(IOMB_ERR_UNSUPPORTED, "silu: leaf is not BF16 or F32");
    }
    const ViewFacts& fx = facts[0];
    if (fx.rows > 0xFFFFFFFFull || fx.cols > 0xFFFFFFFFull) {
        return fail(IOMB_ERR_UNSUPPORTED, "silu: matrix extent exceeds the kernel limit");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint16_t* table = nullptr;
    if (x->dtype == IOMB_BF16) {
        const int status = silu_table(s, &table);
        if (status != IOMB_OK) return status;
    }

    SiluParams p{};
    uint64_t strides[4][kMaxLead] = {};
    for (uint32_t k = 0; k < count; ++k) {
        for (uint32_t axis = 0; axis < fx.leading; ++axis) {
            strides[k][axis] = views[k]->plane_strides[axis];
        }
    }
    collapse_leading(fx.leading, x->dims, strides, count, &p.leading);
    p.x = make_operand(*x, facts[0], strides[0], p.leading, false, false);
    p.out = make_operand(*out, facts[1], strides[1], p.leading, false, false);
    if (fused) p.up = make_operand(*up, facts[2], strides[2], p.leading, false, false);
    if (count == 4) p.activated = make_operand(*activated, facts[3], strides[3], p.leading, false, false);
    p.has_activated = count == 4 ? 1u : 0u;
    p.rows = static_cast<uint32_t>(fx.rows);
    p.cols = static_cast<uint32_t>(fx.cols);
    p.tile_rows = static_cast<uint32_t>(fx.tile_rows);
    p.tile_cols = static_cast<uint32_t>(fx.tile_cols);
    p.items = p.leading.planes * fx.tile_rows * fx.tile_cols;
    p.table = table;

    const bool bf16 = x->dtype == IOMB_BF16;
    const bool linear = p.leading.contiguous && fx.rows % kTile == 0 && fx.cols % kTile == 0;
    if (linear) {
        auto start = [&](uint32_t k) {
            return static_cast<unsigned char*>(views[k]->base) + views[k]->plane_offset * facts[k].plane_bytes;
        };
        const uint4* xs = reinterpret_cast<const uint4*>(start(0));
        uint4* os = reinterpret_cast<uint4*>(start(1));
        const uint4* us = fused ? reinterpret_cast<const uint4*>(start(2)) : nullptr;
        uint4* as = count == 4 ? reinterpret_cast<uint4*>(start(3)) : nullptr;
        const uint64_t vectors = p.leading.planes * fx.plane_bytes / 16;
        // The shared-memory table pays for itself once every SM has a few MiB to do.
        const bool staged = bf16 && vectors * 16 >= (16ull << 20);
        if (staged) {
            auto kernel = fused ? silu_stream_kernel<2, true, true> : silu_stream_kernel<2, false, true>;
            const int prepared = allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
            if (prepared != IOMB_OK) return prepared;
            const uint64_t per_cta = static_cast<uint64_t>(kSiluStagedThreads) * kSiluUnroll;
            kernel<<<grid_for((vectors + per_cta - 1) / per_cta, 1), kSiluStagedThreads,
                     kSiluTableBytes, s>>>(xs, us, as, os, vectors, table);
        } else {
            const uint64_t per_cta = static_cast<uint64_t>(kSiluThreads) * kSiluUnroll;
            const unsigned grid = grid_one_shot((vectors + per_cta - 1) / per_cta);
            if (bf16) {
                if (fused) silu_stream_kernel<2, true, false><<<grid, kSiluThreads, 0, s>>>(xs, us, as, os, vectors, table);
                else silu_stream_kernel<2, false, false><<<grid, kSiluThreads, 0, s>>>(xs, us, as, os, vectors, table);
            } else {
                if (fused) silu_stream_kernel<4, true, false><<<grid, kSiluThreads, 0, s>>>(xs, us, as, os, vectors, table);
                else silu_stream_kernel<4, false, false><<<grid, kSiluThreads, 0, s>>>(xs, us, as, os, vectors, table);
            }
        }
    } else {
        const unsigned grid = grid_one_shot((p.items + kSiluThreads / 32 - 1) / (kSiluThreads / 32));
        if (bf16) {
            if (fused) silu_tiled_kernel<2, true><<<grid, kSiluThreads, 0, s>>>(p);
            else silu_tiled_kernel<2, false><<<grid, kSiluThreads, 0, s>>>(p);
        } else {
            if (fused) silu_tiled_kernel<4, true><<<grid, kSiluThreads, 0, s>>>(p);
            else silu_tiled_kernel<4, false><<<grid, kSiluThreads, 0, s>>>(p);
        }
    }
    return check_launch("silu launch");
}

int prepare_silu(cudaStream_t stream) {
    const uint16_t* table = nullptr;
    int status = silu_table(stream, &table);
    if (status == IOMB_OK) {
        status = allow_full_shared_memory(
                reinterpret_cast<const void*>(silu_stream_kernel<2, true, true>));
    }
    if (status == IOMB_OK) {
        status = allow_full_shared_memory(
                reinterpret_cast<const void*>(silu_stream_kernel<2, false, true>));
    }
    return status;
}

}  // namespace iomb

extern "C" int iomb_silu(const iomb_view* x, const iomb_view* out, void* stream) {
    return iomb::silu_dispatch(x, nullptr, nullptr, out, stream);
}

extern "C" int iomb_silu_mul(const iomb_view* x, const iomb_view* up, const iomb_view* activated,
                             const iomb_view* out, void* stream) {
    if (up == nullptr) {
        return iomb::fail(IOMB_ERR_INVALID_ARGUMENT, "silu_mul: the up operand is required");
    }
    return iomb::silu_dispatch(x, up, activated, out, stream);
}
