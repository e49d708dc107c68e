/*
 * iom_b200 — C ABI of the B200 (sm_100a) device tensor-op kernels for IOM.
 *
 * This is the drop-in boundary: plain pointers, sizes and POD descriptors, no
 * C++ or torch types. Every entry point replaces one device operation of the
 * reference CUDA backend (rlewczuk/iom, src/cuda + src/shared) and takes the
 * same information the reference's backend hooks receive in their value
 * snapshots. Reference citations are paths inside the reference project.
 *
 * Conventions shared by all entry points
 *   - Tensors live in the reference's standard 16x16 tiled layout
 *     (src/tensor.cpp:136-164): leading plane, tile row, tile column, row in
 *     tile, column in tile; both matrix axes padded to multiples of 16. Padding
 *     slots are never read for arithmetic and never written.
 *   - `stream` is a cudaStream_t passed as void*. Launches are asynchronous on
 *     that stream. No entry point allocates, frees or synchronises.
 *   - Return value: IOMB_OK or a positive iomb_status. The codes are the
 *     magnitudes of the reference's negative OidError values
 *     (include/iom/oid.hpp:16-23), so a host layer maps status s to oid -s.
 *     iomb_last_error() returns a thread-local description of the last failure.
 *   - There is no CPU fallback: without a CUDA device every compute entry point
 *     returns IOMB_ERR_DEVICE.
 */
#ifndef IOM_B200_H
#define IOM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IOMB_MAX_RANK 8
#define IOMB_MAX_LEADING 6
#define IOMB_TILE 16

/* Mirrors OidError (include/iom/oid.hpp:16-23) with the sign dropped. */
typedef enum iomb_status {
    IOMB_OK = 0,
    IOMB_ERR_INVALID_ARGUMENT = 1,
    IOMB_ERR_UNSUPPORTED = 2,
    IOMB_ERR_OVERFLOW = 3,
    IOMB_ERR_RESOURCE_EXHAUSTED = 4,
    IOMB_ERR_DEVICE = 5,
    IOMB_ERR_INTERNAL = 6
} iomb_status;

/* Leaf encodings with the ordinals of iom::DataType (include/iom/tensor.hpp:10-32). */
typedef enum iomb_dtype {
    IOMB_BOOL = 0,
    IOMB_I2 = 1, IOMB_U2 = 2, IOMB_I4 = 3, IOMB_U4 = 4,
    IOMB_I8 = 5, IOMB_U8 = 6, IOMB_I16 = 7, IOMB_U16 = 8,
    IOMB_I32 = 9, IOMB_U32 = 10, IOMB_I64 = 11, IOMB_U64 = 12,
    IOMB_F4_E2M1 = 13, IOMB_F6_E2M3 = 14, IOMB_F6_E3M2 = 15,
    IOMB_F8_E4M3FN = 16, IOMB_F8_E5M2 = 17, IOMB_F8_E8M0 = 18,
    IOMB_F16 = 19, IOMB_BF16 = 20, IOMB_F32 = 21, IOMB_F64 = 22
} iomb_dtype;

/* DeviceOps::BinaryOperation (include/iom/iom.hpp:381). */
typedef enum iomb_binary_op {
    IOMB_ADD = 0,
    IOMB_MUL = 1,
    IOMB_SUB = 2,
    IOMB_DIV = 3
} iomb_binary_op;

/*
 * Value snapshot of one tensor view: what BinaryViewSnapshot / CopyViewSnapshot /
 * CacheAppendViewSnapshot carry (include/iom/iom.hpp:382-426).
 *   base           owner storage (device pointer, at least 32-byte aligned)
 *   storage_bytes  bytes the owner reserves (TensorSpec::tiled_storage_nbytes)
 *   dims           full logical shape, rank 2..8; dims[rank-2], dims[rank-1]
 *                  are the owner's matrix extents (views never transform them)
 *   plane_offset,
 *   plane_strides  in whole owner planes, one stride per leading axis
 */
typedef struct iomb_view {
    void* base;
    uint64_t storage_bytes;
    uint32_t dtype;
    uint32_t rank;
    uint64_t dims[IOMB_MAX_RANK];
    uint64_t plane_offset;
    uint64_t plane_strides[IOMB_MAX_LEADING];
} iomb_view;

/* RMSNorm accumulation order (see iomb_rmsnorm). */
typedef enum iomb_rms_order {
    /* 16 column accumulators per row, each summed in tile order, then the fixed
     * tree ((l0+l4)+l8)+l12 ... of src/cpu/avx512_bf16_rmsnorm_reduction.cpp:69-81.
     * Bit-identical to the reference's AVX-512 BF16 CPU build for BF16. */
    IOMB_RMS_LANES16 = 0,
    /* One accumulator per row walking the features in order: the portable CPU
     * recurrence (src/cpu/queue.cpp:1187-1196). Bit-identical to it. Slower. */
    IOMB_RMS_SEQUENTIAL = 1
} iomb_rms_order;

const char* iomb_last_error(void);

/* The kernel instance the calling thread's most recent iomb_rmsnorm / iomb_add_rmsnorm
 * launched, with the template arguments its dispatcher chose (for benchmark records);
 * empty before the first such call. No counterpart in the reference. */
const char* iomb_last_launch(void);

/* The long-row RMSNorm kernels wait for their asynchronous copies a bounded number of
 * polls. A launch in which a wait gave up (never expected: its results are incomplete)
 * adds one per CTA to a device counter; this reads it (synchronous, after the launches of
 * interest have completed). */
int iomb_rmsnorm_copy_timeouts(unsigned int* count);

/* Library/ABI version, bumped when a struct or signature changes. */
uint32_t iomb_abi_version(void);

/* Pure helpers of the layout contract (no device needed). */
uint32_t iomb_dtype_bits(uint32_t dtype);                 /* detail::leaf_bits, src/tensor.cpp:107-134 */
int iomb_tiled_storage_nbytes(const uint64_t* dims, uint32_t rank, uint32_t dtype,
                              uint64_t* out_bytes);      /* TensorSpec::tiled_storage_nbytes, src/tensor.cpp:95-102 */
int iomb_logical_nbytes(const uint64_t* dims, uint32_t rank, uint32_t dtype,
                        uint64_t* out_bytes);            /* TensorSpec::logical_nbytes, src/tensor.cpp:88-93 */
uint64_t iomb_plane_slot(uint64_t rows, uint64_t columns, uint64_t plane,
                         uint64_t row, uint64_t column); /* detail::standard_plane_slot, src/tensor.cpp:136-164 */

/*
 * out = lhs (+|*|-|/) rhs with right-aligned broadcasting.
 * Replaces GpuQueue::binary_impl + grid_stride_binary_kernel / alias_safe_binary_kernel
 * (src/shared/gpu_queue_operations.inl:65-124,756-818; src/shared/standard_tiled_add.inl:206-464);
 * admission rules of DeviceOps::validate_binary (src/device_ops_binary.cpp:102-181).
 * Leaves: I32/U32, F32, BF16 on the vector kernels; I8/U8, I16/U16, I64/U64, F16, F8_E4M3FN and
 * F8_E5M2 on a per-element kernel; I2/U2, I4/U4, F4_E2M1, F6_E2M3, F6_E3M2 on a kernel that
 * owns whole tile rows (padding bits survive); F64 on the per-element kernel. Every numeric
 * leaf of the reference.
 * Integers wrap and have no division (src/device_ops_binary.cpp:46-57).
 * Arithmetic equals the scalar codec (src/shared/scalar_binary_codec.hpp:120-178):
 * IEEE binary32 op (division correctly rounded), one RNE encode, every NaN result is
 * the positive quiet NaN (0x7FC00000 / 0x7FC0). BF16 ADD/SUB/MUL may run as packed
 * BF16 instructions (exact result, one rounding): the same codes.
 * F64: one IEEE binary64 operation, the carrier of the reference's GPU kernels
 * (src/shared/standard_tiled_add.inl:110-116); the reference CPU backend's x87 carrier
 * rounds twice and can differ from it by one code.
 * Exact in-place alias (out is the same view as an input) is allowed.
 */
int iomb_binary(int op, const iomb_view* lhs, const iomb_view* rhs,
                const iomb_view* out, void* stream);

/* 1 when iomb_binary serves the leaf (every numeric leaf: all but BOOL and F8_E8M0), else 0.
 * Lets a backend's binary_impl refuse a leaf before a sequence is taken
 * (src/device_ops_binary.cpp:170-177). */
int iomb_binary_supported(uint32_t dtype);

/*
 * One-time set-up of the library on the current device, on `stream`: raises the
 * shared-memory limits of the kernels that need it and builds the BF16 SiLU table, so that
 * no later call does either. Optional (every entry point still does its own set-up on first
 * use); a backend calls it when it constructs its device, before any stream capture. No
 * counterpart in the reference (its kernels need no set-up).
 */
int iomb_prepare_device(void* stream);

/*
 * out[..., r, :] = x[..., r, :] / sqrt(mean(x[..., r, :]^2) + eps) * scale[0, :]
 * Replaces GpuQueue::rmsnorm_impl + standard_tiled_rmsnorm_kernel
 * (src/shared/gpu_queue_operations.inl:206-267,841-869; src/shared/standard_tiled_rmsnorm.inl:437-637);
 * arithmetic of rmsnorm_plane (src/cpu/queue.cpp:1145-1244): FP32 sum of rounded
 * squares, sum/F, +eps, 1/sqrtf (true division), (x*inv)*w, NaN sign cleared,
 * one RNE encode. Leaves: BF16, F32. `order` is an iomb_rms_order. Any row length is
 * served (the reference admits any F): rows of up to 2048 values and the sequential order
 * by a kernel that stages whole row groups in shared memory, longer rows in the lane order
 * by a pipelined kernel that fetches with bulk tensor copies (a call may then issue several
 * launches on `stream`, see iomb_last_launch), rows beyond either one's shared memory from
 * global memory directly. The output shares no owner with an input
 * (src/device_ops_rmsnorm.cpp:75-127).
 */
int iomb_rmsnorm(const iomb_view* x, const iomb_view* scale, const iomb_view* out,
                 float eps, int order, void* stream);

/*
 * Fused residual add + RMSNorm: sum = x + residual (stored, rounded to the leaf),
 * out = rmsnorm(sum, scale). Results equal iomb_binary(ADD) followed by
 * iomb_rmsnorm on the stored sum; the rounded residual is always materialised
 * (docs/ARCHITECTURE.md:465-476). No counterpart in the reference: its session
 * issues the two operations separately (src/session.cpp:2500-2503,1996-2000).
 * `sum` may alias `x` or `residual` exactly; `out` must not alias anything.
 */
int iomb_add_rmsnorm(const iomb_view* x, const iomb_view* residual,
                     const iomb_view* scale, const iomb_view* sum,
                     const iomb_view* out, float eps, int order, void* stream);

/*
 * Bit-exact copy between two views of identical specification.
 * Replaces GpuQueue copy path + grid_stride_copy_kernel
 * (src/shared/standard_tiled_copy_metadata.inl:177-282; admission src/device_ops_copy.cpp:17-52).
 * Any byte-multiple leaf (8/16/32/64 bits) and the leaves of 2, 4 and 6 bits (the bits of
 * padding slots are preserved). An identical window is a no-op.
 */
int iomb_copy(const iomb_view* source, const iomb_view* destination, void* stream);

/*
 * BF16 <-> F32 conversion between views of identical logical shape.
 * No counterpart operation in the reference; semantics are the scalar codec's
 * decode/encode (src/shared/scalar_binary_codec.hpp:45-108): BF16->F32 exact
 * widening, F32->BF16 round-to-nearest-even with overflow to infinity and
 * gradual underflow; a NaN converts to the positive quiet NaN of the target.
 */
int iomb_cast(const iomb_view* source, const iomb_view* destination, void* stream);

/*
 * out = x * sigmoid(x), elementwise, between views of identical shape and leaf.
 * Replaces GpuQueue::silu_impl + silu_kernel (src/cuda/copy.cu:452-596); admission
 * rules of validate_silu (src/device_ops_neural.cpp:362-434: equal shapes and
 * specifications, the output shares neither an owner nor a byte with the input).
 * Arithmetic is scalar_silu on the FP64 carrier of the reference's GPU backends
 * (src/shared/scalar_silu.hpp:66-101, src/cuda/copy.cu:498-503): decode, evaluate
 * the stable form, one RNE encode, canonical NaN. Leaves: BF16, F32. For BF16 the
 * result equals the reference CPU backend's FP32 evaluation for every one of the
 * 65 536 codes. The first BF16 call on a device builds a 128 KiB table inside the
 * library and waits for it once: make it before any stream capture.
 */
int iomb_silu(const iomb_view* x, const iomb_view* out, void* stream);

/*
 * out = silu(x) * up; `activated` (may be NULL) receives silu(x) when given.
 * The decoder MLP's SiLU(gate) followed by the multiply with the up projection
 * (src/session.cpp:2020-2030) in one pass. Results equal iomb_silu followed by
 * iomb_binary(IOMB_MUL) bit for bit (the activated value is rounded to the leaf
 * before the product). Written views share no owner and no byte with any other
 * operand.
 */
int iomb_silu_mul(const iomb_view* x, const iomb_view* up, const iomb_view* activated,
                  const iomb_view* out, void* stream);

/*
 * Fills the rotary angle table on the HOST: for r in [0, rows) and c in [0, width/2),
 * cos_sin[(r * width/2 + c) * 2 + {0,1}] = {cos, sin} of
 * float(first_position + r) * powf(float(theta), float(-2c / width)),
 * the expression of rope_angle (src/cpu/queue.cpp:1356-1367) with the C library's
 * powf / sinf / cosf, which is what fixes the reference CPU backend's bits. No device
 * work. The caller keeps the table in device memory (a rotary cache) for iomb_rope.
 */
int iomb_rope_angles(float* cos_sin, uint64_t first_position, uint64_t rows, uint64_t width,
                     double theta);

/*
 * Split-half rotary embedding: x, out are [..., H, R, W] (rank 3..8, W even); row r sits
 * at position a + r; (out[c], out[c + W/2]) = rotation of (x[c], x[c + W/2]) by the
 * angle of (position, c); a row at position 0 is copied raw.
 * Replaces GpuQueue::rope_impl + src/shared/standard_tiled_rope.inl:83-624; admission rules
 * of validate_rope (src/device_ops_neural.cpp:169-197,241-360: equal shapes, even width,
 * a + R - 1 < 2^24, the output shares neither an owner nor a byte with the input);
 * arithmetic of rope_pair (src/cpu/queue.cpp:1369-1411): four separately rounded FP32
 * products, one subtraction, one addition, one RNE encode each, canonical NaN.
 * `cos_sin` is the DEVICE copy of iomb_rope_angles(first_position = a, rows >= R, W, theta)
 * (or a pointer to row a of a longer table). Leaves: BF16, F32. With the table built on
 * the same host, results are bit-identical to the reference CPU backend.
 */
int iomb_rope(const iomb_view* x, const iomb_view* out, uint64_t a, const float* cos_sin,
              void* stream);

/*
 * out[b, r, f] = table[indices[b, 0, r], f] (raw bits).
 * Replaces GpuQueue::embedding_impl + embedding_word_kernel and its status protocol
 * (src/shared/standard_tiled_embedding.inl:117-199; src/shared/gpu_queue_operations.inl:870-919;
 * admission src/device_ops_embedding.cpp:93-162). `status` points at a 4-byte
 * device word inside the caller's {32,32} workspace: the call resets it to 0 in
 * stream order and the kernel sets it to 1 when any index is negative or >= V;
 * such rows are not written and no table address is formed for them.
 * Payload: byte-multiple leaves and the leaves of 2, 4 and 6 bits. Index: every integer leaf
 * (I2/U2, I4/U4, I8..U64), compared at full width (src/device_ops_embedding.cpp:27-46).
 */
int iomb_embedding(const iomb_view* table, const iomb_view* indices,
                   const iomb_view* out, uint32_t* status, void* stream);

/*
 * destination[..., h, a + r, d] = source[..., h, r, d] (raw bits); only the
 * appended rows are touched.
 * Replaces cache_append_kernel (src/cuda/copy.cu:111-338); admission
 * src/device_ops_cache_append.cpp:157-269 (a <= C, R <= C - a). Byte-multiple leaves and the
 * leaves of 2, 4 and 6 bits.
 */
int iomb_cache_append(const iomb_view* source, const iomb_view* destination,
                      uint64_t a, void* stream);

/*
 * Batched variant with one row offset per index of the first leading axis:
 * destination[b, ..., a[b] + r, d] = source[b, ..., r, d]. `positions` is a
 * device array of dims[0] uint32 values. `status` (device word) is reset to 0
 * and set to 1 when some a[b] + R exceeds the cache length; that b is skipped.
 * No counterpart in the reference, whose call carries one scalar offset
 * (include/iom/iom.hpp:179-185); results equal dims[0] reference calls on
 * select(0, b) views.
 */
int iomb_cache_append_batched(const iomb_view* source, const iomb_view* destination,
                              const uint32_t* positions, uint32_t* status, void* stream);

/*
 * Whole-view sum of squares in FP32 with a fixed, launch-independent order.
 * No counterpart in the reference. `scratch` holds iomb_sumsq_scratch_bytes()
 * bytes of device memory (per-CTA partials); `result` receives one float.
 * Leaves: BF16, F32.
 */
uint64_t iomb_sumsq_scratch_bytes(void);
int iomb_sumsq(const iomb_view* x, void* scratch, float* result, void* stream);

/*
 * iomb_sumsq for callers that cannot provide scratch memory. It has no
 * counterpart in the reference. Who needs it: a backend hook whose operation
 * is admitted with a {0,1} workspace requirement (the caller hands over
 * nothing) while IOM's contract forbids any native allocation after device
 * set-up, or any host that calls in while its memory pools are frozen. The
 * partial sums go to a 16 KiB array built into the library (every GPU that
 * loads the library keeps it until the process exits); the call itself
 * allocates and frees nothing.
 *   - Limit: views of at most IOMB_SUMSQ_STATIC_MAX_ELEMENTS (2^32) elements;
 *     larger views are rejected with IOMB_ERR_INVALID_ARGUMENT.
 *   - The first call on each device looks up the array's device address. Make
 *     that first call during start-up, before any stream capture begins.
 *   - All calls share the one array and it keeps whatever the previous call
 *     left; each call resets what it relies on. Two calls that overlap on the
 *     GPU (different streams, no ordering) race on it: serialise them.
 * Result and leaves are those of iomb_sumsq.
 */
#define IOMB_SUMSQ_STATIC_MAX_ELEMENTS (1ull << 32)
int iomb_sumsq_static(const iomb_view* x, float* result, void* stream);

/*
 * Host-layout <-> tiled conversion on the device.
 * Replaces scatter_plane_kernel / gather_plane_kernel and their per-plane launch
 * loops (src/shared/standard_tiled_copy.inl:286-441). `staging` is a device
 * buffer holding the view's logical row-major payload (exactly
 * logical_nbytes, LSB-first packed; include/iom/tensor.hpp:330-342).
 * Byte-multiple leaves (BOOL is one byte per value) and the leaves of 2, 4 and 6 bits.
 */
int iomb_scatter(const iomb_view* destination, const void* staging, void* stream);
int iomb_gather(const iomb_view* source, void* staging, void* stream);

/*
 * The stages of causal grouped-query attention that are not matrix products. They work on
 * the two fixed workspace segments of the reference's CUDA backend
 * (SdpaNonmatrixRequest, src/cuda/sdpa_nonmatrix_request.hpp:22-49): `scores`, FP32
 * [planes, Hq, Rp, Lp], and `probability`, BF16 of the same extents, Rp = pad16(R),
 * Lp = pad16(L), row-major, both 32-byte aligned and disjoint. Row r of every head sees the
 * tokens t < min(L, a + r + 1). Admission as validate_geometry
 * (src/cuda/sdpa_nonmatrix.cu:82-229): nonzero extents, L <= C, a < C, R <= C - a,
 * Hq % Hkv == 0.
 */
typedef struct iomb_sdpa_stages {
    float* scores;
    void* probability;
    uint64_t planes, Hq, Hkv, R, C, D, a, L;
} iomb_sdpa_stages;

/*
 * scores[p,h,r,t] = scores[p,h,r,t] * (1 / sqrtf(D)) for the visible tokens, a product that
 * is zero stored as +0; every other cell (masked, t >= L, r >= R) keeps its bytes.
 * Replaces launch_sdpa_scale_mask / scale_mask_kernel (src/cuda/sdpa_nonmatrix.cu:347-371).
 */
int iomb_sdpa_scale_mask(const iomb_sdpa_stages* stages, void* stream);

/*
 * probability[p,h,r,t] for t < L from the scores of the visible tokens, everything else
 * untouched. Replaces launch_sdpa_softmax / softmax_kernel (src/cuda/sdpa_nonmatrix.cu:373-477)
 * with the same FP32 steps in the same order: a NaN among the visible scores, or only
 * -inf, makes the visible cells the quiet NaN 0x7FC0; +inf scores share 1/count and the
 * rest are +0; otherwise m = max of the finite scores, sum = expf(s - m) added in token
 * order starting from +0, cell = BF16_RNE(expf(s - m) / sum) with true division; a
 * subnormal quotient rounds to a subnormal BF16. Masked cells t < L are +0.
 */
int iomb_sdpa_softmax(const iomb_sdpa_stages* stages, void* stream);

/*
 * Both stages in one pass over the scores: results equal iomb_sdpa_scale_mask followed by
 * iomb_sdpa_softmax bit for bit. With keep_scores != 0 the scaled scores are also stored
 * (the workspace then equals the two-stage pipeline's); with 0 the scores segment is only
 * read. No counterpart in the reference, which launches the two stages separately.
 */
int iomb_sdpa_scale_mask_softmax(const iomb_sdpa_stages* stages, int keep_scores, void* stream);

/*
 * Canonical stored zeros and NaNs in the merged attention output `out`, a BF16 view
 * [B..., R, Hq*D]: -0 becomes +0, every NaN becomes 0x7FC0; tile padding is not touched.
 * Replaces launch_sdpa_canonicalize_output / canonicalize_output_kernel
 * (src/cuda/sdpa_nonmatrix.cu:479-507).
 */
int iomb_sdpa_canonicalize_output(const iomb_view* out, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* IOM_B200_H */
