/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * Plain-C CPU restatement of the reference's (rlewczuk/iom) device tensor-op
 * path, operating on host copies of the tiled storage. Only tests, the smoke
 * check and the bench's cpu_baseline leg may load this library; the product
 * never does.
 *
 * Pinning: tests/test_oracle_vs_reference.py runs this restatement against the
 * unmodified reference CPU backend (oracle/_ref, built by the Makefile beside
 * this file) and against the golden vectors committed under tests/golden/.
 */
#ifndef IOM_ORACLE_H
#define IOM_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same field layout as the product's view descriptor, defined independently. */
typedef struct iomo_view {
    void* base;               /* host copy of the owner's tiled storage */
    uint64_t storage_bytes;
    uint32_t dtype;           /* iom::DataType ordinal */
    uint32_t rank;
    uint64_t dims[8];
    uint64_t plane_offset;
    uint64_t plane_strides[6];
} iomo_view;

uint32_t iomo_leaf_bits(uint32_t dtype);
uint64_t iomo_plane_slot(uint64_t rows, uint64_t columns, uint64_t plane,
                         uint64_t row, uint64_t column);
uint64_t iomo_tiled_storage_nbytes(const uint64_t* dims, uint32_t rank, uint32_t dtype);
uint64_t iomo_logical_nbytes(const uint64_t* dims, uint32_t rank, uint32_t dtype);

/* op: 0 add, 1 mul, 2 sub, 3 div. The codec with the x87 long double carrier. */
uint64_t iomo_scalar_binary(int op, uint32_t dtype, uint64_t a, uint64_t b);
/* Plain IEEE binary32 arithmetic + canonical NaN, for I32/U32/F32/BF16 add/mul. */
uint64_t iomo_scalar_binary_ieee(int op, uint32_t dtype, uint64_t a, uint64_t b);
uint64_t iomo_codec_mismatches(int op, uint32_t dtype, const void* a, uint64_t na,
                               const void* b, uint64_t nb);
uint64_t iomo_decode_encode(uint32_t src_dtype, uint32_t dst_dtype, uint64_t raw);

/* Each returns 0 on success, 1 for invalid arguments. `ieee` selects the fast
 * arithmetic (valid for I32/U32/F32/BF16 only) instead of the codec. */
int iomo_binary(int op, const iomo_view* lhs, const iomo_view* rhs,
                const iomo_view* out, int ieee);
/* order 0: 16-lane accumulators + fixed tree for BF16 rows without inf/NaN
 * (the reference's AVX-512 BF16 build); order 1: sequential recurrence. */
int iomo_rmsnorm(const iomo_view* x, const iomo_view* scale, const iomo_view* out,
                 float eps, int order);
/* SiLU (src/shared/scalar_silu.hpp:66-101). carrier 0: FP32 evaluation with the C
 * library's expf (the reference CPU backend); carrier 1: FP64 evaluation (the
 * reference's GPU backends, src/cuda/copy.cu:498-503). */
uint64_t iomo_scalar_silu(uint32_t dtype, uint64_t raw, int carrier);
int iomo_silu(const iomo_view* x, const iomo_view* y, int carrier);
/* RoPE (src/cpu/queue.cpp:1338-1592), FP32 carrier, the C library's powf/sinf/cosf. */
void iomo_rope_angle(uint64_t column, uint64_t width, uint64_t position, float theta,
                     float* sine, float* cosine);
int iomo_rope(const iomo_view* x, const iomo_view* out, uint64_t a, double theta);
int iomo_copy(const iomo_view* source, const iomo_view* destination);
int iomo_cast(const iomo_view* source, const iomo_view* destination);
/* *status = 1 and nothing is written when any index is negative or >= V. */
int iomo_embedding(const iomo_view* table, const iomo_view* indices,
                   const iomo_view* out, uint32_t* status);
int iomo_cache_append(const iomo_view* source, const iomo_view* destination, uint64_t a);
double iomo_sumsq(const iomo_view* x);
/* Logical row-major LSB-first packed payload <-> tiled storage. */
int iomo_scatter(const iomo_view* destination, const void* logical);
int iomo_gather(const iomo_view* source, void* logical);

/*
 * The attention stages that are not matrix products, on host copies of the two workspace
 * segments (FP32 scores and BF16 probability, both [planes, Hq, pad16(R), pad16(L)]):
 * the steps of src/cuda/sdpa_nonmatrix.cu:347-507 one for one, with the C library's expf,
 * which is also what the reference CPU backend's softmax calls (src/cpu/sdpa.cpp:258-300).
 * Pinned by the known answers of the reference's stage test
 * (test/cuda/test_cuda_sdpa_nonmatrix.cpp) on the CPU, and on a GPU against the
 * reference's own stage kernels compiled into oracle/_ref.
 */
typedef struct iomo_sdpa_stages {
    float* scores;
    uint16_t* probability;
    uint64_t planes, Hq, Hkv, R, C, D, a, L;
} iomo_sdpa_stages;
int iomo_sdpa_scale_mask(const iomo_sdpa_stages* stages);
int iomo_sdpa_softmax(const iomo_sdpa_stages* stages);
int iomo_sdpa_canonicalize_output(const iomo_view* out);

#ifdef __cplusplus
}
#endif
#endif
