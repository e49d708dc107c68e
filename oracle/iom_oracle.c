/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * Plain-C CPU restatement of the reference's (rlewczuk/iom) device tensor-op
 * path. Every function cites the reference file:line whose behaviour it
 * restates. It works on host copies of the standard 16x16 tiled storage.
 *
 * Parity pin: tests/test_oracle_vs_reference.py compares this file, byte for
 * byte of physical storage, with the unmodified reference CPU backend
 * (portable and AVX-512 BF16 builds, oracle/_ref) and with tests/golden/.
 *
 * Build: see Makefile (gcc -std=c11 -O2 -ffp-contract=off, no fast-math).
 */
#include "iom_oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define TILE 16u
#define TILE_SLOTS 256u

enum {
    DT_BOOL = 0, DT_I2, DT_U2, DT_I4, DT_U4, DT_I8, DT_U8, DT_I16, DT_U16,
    DT_I32, DT_U32, DT_I64, DT_U64, DT_F4_E2M1, DT_F6_E2M3, DT_F6_E3M2,
    DT_F8_E4M3FN, DT_F8_E5M2, DT_F8_E8M0, DT_F16, DT_BF16, DT_F32, DT_F64
};

/* detail::leaf_bits, src/tensor.cpp:107-134. 0 for an unknown ordinal. */
uint32_t iomo_leaf_bits(uint32_t dtype) {
    switch (dtype) {
        case DT_BOOL: return 8;
        case DT_I2: case DT_U2: return 2;
        case DT_I4: case DT_U4: case DT_F4_E2M1: return 4;
        case DT_F6_E2M3: case DT_F6_E3M2: return 6;
        case DT_I8: case DT_U8: case DT_F8_E4M3FN: case DT_F8_E5M2:
        case DT_F8_E8M0: return 8;
        case DT_I16: case DT_U16: case DT_F16: case DT_BF16: return 16;
        case DT_I32: case DT_U32: case DT_F32: return 32;
        case DT_I64: case DT_U64: case DT_F64: return 64;
        default: return 0;
    }
}

/* detail::standard_plane_slot, src/tensor.cpp:136-164. */
uint64_t iomo_plane_slot(uint64_t rows, uint64_t columns, uint64_t plane,
                         uint64_t row, uint64_t column) {
    const uint64_t tile_rows = (rows + TILE - 1) / TILE;
    const uint64_t tile_columns = (columns + TILE - 1) / TILE;
    const uint64_t tile_index =
            plane * (tile_rows * tile_columns) + (row / TILE) * tile_columns + column / TILE;
    return tile_index * TILE_SLOTS + (row % TILE) * TILE + column % TILE;
}

/* TensorSpec::tiled_storage_nbytes, src/tensor.cpp:76-102. */
uint64_t iomo_tiled_storage_nbytes(const uint64_t* dims, uint32_t rank, uint32_t dtype) {
    uint64_t elements = 1;
    for (uint32_t i = 0; i + 2 < rank; ++i) elements *= dims[i];
    elements *= (dims[rank - 2] + TILE - 1) / TILE * TILE;
    elements *= (dims[rank - 1] + TILE - 1) / TILE * TILE;
    return (elements * iomo_leaf_bits(dtype) + 7) / 8;
}

/* TensorSpec::logical_nbytes, src/tensor.cpp:88-93. */
uint64_t iomo_logical_nbytes(const uint64_t* dims, uint32_t rank, uint32_t dtype) {
    uint64_t elements = 1;
    for (uint32_t i = 0; i < rank; ++i) elements *= dims[i];
    return (elements * iomo_leaf_bits(dtype) + 7) / 8;
}

/* cpu_detail::load_bits / store_bits, src/cpu/transfer_helpers.hpp:14-40
 * (LSB-first bit addressing), with whole-byte shortcuts. */
static uint64_t load_bits(const unsigned char* base, uint64_t bit, uint32_t nbits) {
    if ((nbits & 7u) == 0 && (bit & 7u) == 0) {
        uint64_t value = 0;
        memcpy(&value, base + bit / 8, nbits / 8); /* little-endian host */
        return value;
    }
    uint64_t value = 0;
    for (uint32_t i = 0; i < nbits; ++i) {
        const uint64_t b = bit + i;
        value |= (uint64_t)((base[b / 8] >> (b % 8)) & 1u) << i;
    }
    return value;
}

static void store_bits(unsigned char* base, uint64_t bit, uint32_t nbits, uint64_t value) {
    if ((nbits & 7u) == 0 && (bit & 7u) == 0) {
        memcpy(base + bit / 8, &value, nbits / 8);
        return;
    }
    for (uint32_t i = 0; i < nbits; ++i) {
        const uint64_t b = bit + i;
        const unsigned char mask = (unsigned char)(1u << (b % 8));
        if ((value >> i) & 1u) base[b / 8] |= mask;
        else base[b / 8] &= (unsigned char)~mask;
    }
}

/* ---- scalar codec: src/shared/scalar_binary_codec.hpp ------------------ */

typedef struct {
    unsigned bits, ebits, fbits;
    int bias;
    int finite_only, infs;
} format_t;

/* Codec::format, scalar_binary_codec.hpp:30-43. */
static format_t format_of(uint32_t dtype) {
    switch (dtype) {
        case DT_F4_E2M1: return (format_t){4, 2, 1, 1, 1, 0};
        case DT_F6_E2M3: return (format_t){6, 2, 3, 1, 1, 0};
        case DT_F6_E3M2: return (format_t){6, 3, 2, 3, 1, 0};
        case DT_F8_E4M3FN: return (format_t){8, 4, 3, 7, 1, 0};
        case DT_F8_E5M2: return (format_t){8, 5, 2, 15, 0, 1};
        case DT_F16: return (format_t){16, 5, 10, 15, 0, 1};
        case DT_BF16: return (format_t){16, 8, 7, 127, 0, 1};
        case DT_F32: return (format_t){32, 8, 23, 127, 0, 1};
        case DT_F64: return (format_t){64, 11, 52, 1023, 0, 1};
        default: return (format_t){0, 0, 0, 0, 0, 0};
    }
}

/* Codec::decode, scalar_binary_codec.hpp:45-65 (host carrier: long double,
 * src/shared/scalar_add.hpp:15-16). */
static long double codec_decode(uint64_t raw, format_t f) {
    const uint64_t sign = raw >> (f.ebits + f.fbits);
    const uint64_t emask = ((uint64_t)1 << f.ebits) - 1;
    const uint64_t frac = raw & (((uint64_t)1 << f.fbits) - 1);
    const uint64_t exp = (raw >> f.fbits) & emask;
    if (exp == emask && (!f.finite_only || f.ebits >= 4)) {
        if (f.infs && frac == 0) return sign ? -(long double)INFINITY : (long double)INFINITY;
        return (long double)NAN;
    }
    const long double value = exp
            ? ldexpl((long double)(((uint64_t)1 << f.fbits) + frac),
                     (int)exp - f.bias - (int)f.fbits)
            : ldexpl((long double)frac, 1 - f.bias - (int)f.fbits);
    return sign ? -value : value;
}

/* Codec::round_even, scalar_binary_codec.hpp:110-118. */
static uint64_t codec_round_even(long double value) {
    const long double integral = floorl(value);
    const long double remainder = value - integral;
    return (uint64_t)integral
            + (uint64_t)(remainder > 0.5L
                         || (remainder == 0.5L && ((uint64_t)integral & 1u)));
}

/* Codec::encode, scalar_binary_codec.hpp:67-108. */
static uint64_t codec_encode(long double value, format_t f) {
    const uint64_t sign = signbit(value) ? 1 : 0;
    value = fabsl(value);
    const uint64_t emask = ((uint64_t)1 << f.ebits) - 1;
    const uint64_t fmask = ((uint64_t)1 << f.fbits) - 1;
    const uint64_t finite_emax = (f.finite_only && f.ebits < 4) ? emask : emask - 1;
#define PACK(e, m) ((sign << (f.ebits + f.fbits)) | ((uint64_t)(e) << f.fbits) | (uint64_t)(m))
    const uint64_t overflow = f.infs ? PACK(emask, 0) : PACK(finite_emax, fmask);
    if (isnan(value)) {
        if (f.finite_only && f.ebits < 4) value = LDBL_MAX;
        else return PACK(emask, f.finite_only ? fmask : (uint64_t)1 << (f.fbits - 1));
    }
    if (isinf(value)) return overflow;
    if (value == 0) return sign << (f.ebits + f.fbits);
    const int min_sub = 1 - f.bias - (int)f.fbits;
    const int max_exp = (int)finite_emax - f.bias;
    int exponent = 0;
    (void)frexpl(value, &exponent);
    --exponent;
    if (exponent < min_sub + (int)f.fbits) {
        const uint64_t q = codec_round_even(ldexpl(value, -min_sub));
        return q == ((uint64_t)1 << f.fbits) ? PACK(1, 0) : PACK(0, q);
    }
    if (exponent > max_exp) return overflow;
    uint64_t fraction = codec_round_even(
            ldexpl(value, (int)f.fbits - exponent) - (long double)((uint64_t)1 << f.fbits));
    if (fraction == ((uint64_t)1 << f.fbits)) {
        ++exponent;
        fraction = 0;
    }
    if (exponent > max_exp) return overflow;
    return PACK((uint64_t)(exponent + f.bias), fraction);
#undef PACK
}

/* Codec::arithmetic, scalar_binary_codec.hpp:120-148. */
static long double codec_arithmetic(int op, long double x, long double y) {
    if (isnan(x) || isnan(y)) return (long double)NAN;
    switch (op) {
        case 0:
            if (isinf(x) && isinf(y) && (signbit(x) != 0) != (signbit(y) != 0))
                return (long double)NAN;
            if (x == 0 && y == 0) return (signbit(x) && signbit(y)) ? -0.0L : 0.0L;
            {
                const long double result = x + y;
                return result == 0 ? 0.0L : result;
            }
        case 1:
            if ((isinf(x) && y == 0) || (isinf(y) && x == 0)) return (long double)NAN;
            return x * y;
        case 2:
            if (isinf(x) && isinf(y) && (signbit(x) != 0) == (signbit(y) != 0))
                return (long double)NAN;
            return x - y;
        default:
            if ((x == 0 && y == 0) || (isinf(x) && isinf(y))) return (long double)NAN;
            return x / y;
    }
}

/* Codec::integer_width, scalar_binary_codec.hpp:150-161. */
static unsigned integer_width(uint32_t dtype) {
    switch (dtype) {
        case DT_I2: case DT_U2: return 2;
        case DT_I4: case DT_U4: return 4;
        case DT_I8: case DT_U8: return 8;
        case DT_I16: case DT_U16: return 16;
        case DT_I32: case DT_U32: return 32;
        case DT_I64: case DT_U64: return 64;
        default: return 0;
    }
}

/* Codec::binary, scalar_binary_codec.hpp:163-178. */
uint64_t iomo_scalar_binary(int op, uint32_t dtype, uint64_t a, uint64_t b) {
    const unsigned width = integer_width(dtype);
    if (width) {
        if (op == 3) return 0;
        const uint64_t mask = width == 64 ? ~(uint64_t)0 : (((uint64_t)1 << width) - 1);
        if (op == 0) return (a + b) & mask;
        if (op == 1) return (a * b) & mask;
        return (a - b) & mask;
    }
    const format_t f = format_of(dtype);
    if (!f.bits) return 0;
    return codec_encode(codec_arithmetic(op, codec_decode(a, f), codec_decode(b, f)), f);
}

static float bits_to_float(uint32_t bits) {
    float value;
    memcpy(&value, &bits, sizeof value);
    return value;
}

static uint32_t float_to_bits(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof bits);
    return bits;
}

/* Round-to-nearest-even of a non-NaN binary32 to BF16: the integer form the
 * reference's AVX path uses (src/cpu/avx512_bf16_binary_add_sub.cpp:68-75). */
static uint32_t float_to_bf16_rne(float value) {
    const uint32_t bits = float_to_bits(value);
    if (isnan(value)) return 0x7FC0u;
    return (bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16;
}

/* The arithmetic the kernels implement: one IEEE binary32 add/mul/sub/div
 * (rounded once), then one RNE encode for BF16, every NaN result canonical.
 * Equal to iomo_scalar_binary for the byte-multiple integers, F32, BF16 and F16
 * because rounding a binary32 (or x87) result again to a format with at most
 * (p - 2) / 2 significand bits is innocuous for all four operations (F16: 11 bits
 * against 24); tests/test_layout_and_codec.py proves
 * the equality exhaustively for BF16 and on boundary-rich samples for F32.
 * Integer division does not exist (the codec answers 0, admission rejects it). */
/* binary16 <-> binary32 with plain integer arithmetic (no compiler half type):
 * exact widening, and one round-to-nearest-even narrowing with gradual underflow
 * and overflow to infinity. */
static float half_to_float(uint32_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    const uint32_t exponent = (h >> 10) & 0x1Fu;
    uint32_t mantissa = h & 0x3FFu;
    if (exponent == 0x1Fu) return bits_to_float(sign | 0x7F800000u | (mantissa << 13));
    if (exponent == 0) {
        if (mantissa == 0) return bits_to_float(sign);
        int shift = 0;
        while (!(mantissa & 0x400u)) {
            mantissa <<= 1;
            ++shift;
        }
        return bits_to_float(sign | ((uint32_t)(113 - shift) << 23) | ((mantissa & 0x3FFu) << 13));
    }
    return bits_to_float(sign | ((exponent + 112u) << 23) | (mantissa << 13));
}

static uint32_t float_to_half_rne(float value) {
    const uint32_t bits = float_to_bits(value);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    const uint32_t magnitude = bits & 0x7FFFFFFFu;
    if (magnitude > 0x7F800000u) return 0x7E00u;                   /* canonical positive NaN */
    if (magnitude >= 0x47800000u) return sign | 0x7C00u;           /* >= 2^16: infinity */
    if (magnitude < 0x33000000u) return sign;                      /* < 2^-25: zero */
    const int exponent = (int)(magnitude >> 23) - 127;
    uint32_t significand = (magnitude & 0x7FFFFFu) | 0x800000u;    /* 24 bits */
    int shift = 13;                                                /* normal: keep 11 bits */
    if (exponent < -14) shift += -14 - exponent;                   /* subnormal: quantum 2^-24 */
    uint32_t quotient = significand >> shift;
    const uint32_t remainder = significand & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (remainder > half || (remainder == half && (quotient & 1u))) ++quotient;
    uint32_t code;
    if (exponent >= -14) {
        code = ((uint32_t)(exponent + 15) << 10) + (quotient - 0x400u);
        if (code >= 0x7C00u) code = 0x7C00u;
    } else {
        code = quotient;
    }
    return sign | code;
}

uint64_t iomo_scalar_binary_ieee(int op, uint32_t dtype, uint64_t a, uint64_t b) {
    const unsigned width = integer_width(dtype);
    if (width) {
        /* Integers of every width wrap; division does not exist. */
        if (op == 3) return 0;
        const uint64_t mask = width == 64 ? ~(uint64_t)0 : (((uint64_t)1 << width) - 1);
        return (op == 0 ? a + b : op == 1 ? a * b : a - b) & mask;
    }
    float x, y;
    if (format_of(dtype).bits && format_of(dtype).bits <= 8) {
        /* F4, F6, F8: exact decode, one binary32 operation, one encode: 24 >= 2 * 4 + 2 */
        const format_t f8 = format_of(dtype);
        x = (float)codec_decode(a, f8);
        y = (float)codec_decode(b, f8);
        volatile float r8 = op == 0 ? x + y : op == 1 ? x * y : op == 2 ? x - y : x / y;
        const float narrow = r8;
        return isnan(narrow) ? codec_encode((long double)NAN, f8) : codec_encode((long double)narrow, f8);
    }
    if (dtype == DT_F16) {
        x = half_to_float((uint32_t)a);
        y = half_to_float((uint32_t)b);
        volatile float r16 = op == 0 ? x + y : op == 1 ? x * y : op == 2 ? x - y : x / y;
        return float_to_half_rne(r16);
    }
    if (dtype == DT_BF16) {
        x = bits_to_float((uint32_t)a << 16);
        y = bits_to_float((uint32_t)b << 16);
    } else {
        x = bits_to_float((uint32_t)a);
        y = bits_to_float((uint32_t)b);
    }
    volatile float r = op == 0 ? x + y : op == 1 ? x * y : op == 2 ? x - y : x / y;
    const float result = r;
    if (dtype == DT_BF16) return float_to_bf16_rne(result);
    return isnan(result) ? 0x7FC00000u : float_to_bits(result);
}

/* Counts pairs (a[i], b[j]) on which the codec and the IEEE form disagree. */
uint64_t iomo_codec_mismatches(int op, uint32_t dtype, const void* a, uint64_t na,
                               const void* b, uint64_t nb) {
    const uint32_t bits = iomo_leaf_bits(dtype);
    uint64_t mismatches = 0;
    for (uint64_t i = 0; i < na; ++i) {
        const uint64_t x = bits <= 8 ? ((const uint8_t*)a)[i]
                : bits == 16 ? ((const uint16_t*)a)[i] : ((const uint32_t*)a)[i];
        for (uint64_t j = 0; j < nb; ++j) {
            const uint64_t y = bits <= 8 ? ((const uint8_t*)b)[j]
                    : bits == 16 ? ((const uint16_t*)b)[j] : ((const uint32_t*)b)[j];
            if (iomo_scalar_binary(op, dtype, x, y) != iomo_scalar_binary_ieee(op, dtype, x, y)) {
                ++mismatches;
            }
        }
    }
    return mismatches;
}

/* decode in the source format, encode in the destination format: the cast
 * semantics derived from scalar_binary_codec.hpp:45-108. */
uint64_t iomo_decode_encode(uint32_t src_dtype, uint32_t dst_dtype, uint64_t raw) {
    return codec_encode(codec_decode(raw, format_of(src_dtype)), format_of(dst_dtype));
}

/* ---- view helpers ------------------------------------------------------- */

typedef struct {
    uint64_t rows, columns;
    uint32_t leading;
    uint32_t bits;
} geometry_t;

static int geometry_of(const iomo_view* v, geometry_t* g) {
    if (v == NULL || v->base == NULL || v->rank < 2 || v->rank > 8) return 1;
    g->bits = iomo_leaf_bits(v->dtype);
    if (g->bits == 0) return 1;
    for (uint32_t i = 0; i < v->rank; ++i) {
        if (v->dims[i] == 0) return 1;
    }
    g->leading = v->rank - 2;
    g->rows = v->dims[v->rank - 2];
    g->columns = v->dims[v->rank - 1];
    return 0;
}

static uint64_t leading_count(const iomo_view* v) {
    uint64_t count = 1;
    for (uint32_t i = 0; i + 2 < v->rank; ++i) count *= v->dims[i];
    return count;
}

/* Owner plane of the `index`-th logical plane (row-major over leading dims). */
static uint64_t view_plane(const iomo_view* v, uint64_t index) {
    uint64_t plane = v->plane_offset;
    for (uint32_t axis = v->rank - 2; axis-- > 0;) {
        plane += (index % v->dims[axis]) * v->plane_strides[axis];
        index /= v->dims[axis];
    }
    return plane;
}

static uint64_t element_bit(const iomo_view* v, const geometry_t* g, uint64_t plane,
                            uint64_t row, uint64_t column) {
    (void)v;
    return iomo_plane_slot(g->rows, g->columns, plane, row, column) * g->bits;
}

/* ---- binary: src/cpu/queue.cpp:414-536, src/device_ops_binary.cpp:61-181 -- */

int iomo_binary(int op, const iomo_view* lhs, const iomo_view* rhs,
                const iomo_view* out, int ieee) {
    geometry_t gl, gr, go;
    if (geometry_of(lhs, &gl) || geometry_of(rhs, &gr) || geometry_of(out, &go)) return 1;
    if (lhs->dtype != rhs->dtype || lhs->dtype != out->dtype) return 1;
    if (op < 0 || op > 3) return 1;
    const uint32_t rank = lhs->rank > rhs->rank ? lhs->rank : rhs->rank;
    if (out->rank != rank) return 1;
    uint64_t result[8];
    /* right-aligned broadcast, device_ops_binary.cpp:121-143 */
    for (uint32_t i = 0; i < rank; ++i) {
        const uint64_t la = i < rank - lhs->rank ? 1 : lhs->dims[i - (rank - lhs->rank)];
        const uint64_t ra = i < rank - rhs->rank ? 1 : rhs->dims[i - (rank - rhs->rank)];
        if (la != ra && la != 1 && ra != 1) return 1;
        result[i] = la > ra ? la : ra;
        if (out->dims[i] != result[i]) return 1;
    }
    const uint32_t leading = rank - 2;
    /* logical_plane_strides, device_ops_binary.cpp:61-100: zero on broadcast axes */
    uint64_t stride[3][6];
    const iomo_view* operand[3] = {lhs, rhs, out};
    for (int k = 0; k < 3; ++k) {
        const uint32_t offset = rank - operand[k]->rank;
        for (uint32_t axis = 0; axis < leading; ++axis) {
            stride[k][axis] = 0;
            if (axis < offset) continue;
            const uint32_t source_axis = axis - offset;
            if (operand[k]->dims[source_axis] == 1 && result[axis] != 1) continue;
            stride[k][axis] = operand[k]->plane_strides[source_axis];
        }
    }
    const int lhs_bc_rows = gl.rows == 1 && result[rank - 2] != 1;
    const int rhs_bc_rows = gr.rows == 1 && result[rank - 2] != 1;
    const int lhs_bc_cols = gl.columns == 1 && result[rank - 1] != 1;
    const int rhs_bc_cols = gr.columns == 1 && result[rank - 1] != 1;
    uint64_t planes = 1;
    for (uint32_t i = 0; i < leading; ++i) planes *= result[i];
    const uint32_t bits = go.bits;
    unsigned char* out_base = (unsigned char*)out->base;
    const unsigned char* lhs_base = (const unsigned char*)lhs->base;
    const unsigned char* rhs_base = (const unsigned char*)rhs->base;
    for (uint64_t index = 0; index < planes; ++index) {
        uint64_t plane[3] = {lhs->plane_offset, rhs->plane_offset, out->plane_offset};
        uint64_t rest = index;
        for (uint32_t axis = leading; axis-- > 0;) {
            const uint64_t coordinate = rest % result[axis];
            rest /= result[axis];
            for (int k = 0; k < 3; ++k) plane[k] += coordinate * stride[k][axis];
        }
        for (uint64_t row = 0; row < result[rank - 2]; ++row) {
            for (uint64_t column = 0; column < result[rank - 1]; ++column) {
                const uint64_t a = load_bits(
                        lhs_base,
                        element_bit(lhs, &gl, plane[0], lhs_bc_rows ? 0 : row,
                                    lhs_bc_cols ? 0 : column),
                        bits);
                const uint64_t b = load_bits(
                        rhs_base,
                        element_bit(rhs, &gr, plane[1], rhs_bc_rows ? 0 : row,
                                    rhs_bc_cols ? 0 : column),
                        bits);
                const uint64_t r = ieee ? iomo_scalar_binary_ieee(op, out->dtype, a, b)
                                        : iomo_scalar_binary(op, out->dtype, a, b);
                store_bits(out_base, element_bit(out, &go, plane[2], row, column), bits, r);
            }
        }
    }
    return 0;
}

/* ---- rmsnorm: src/cpu/queue.cpp:1106-1296 -------------------------------- */

/* sum_lanes, src/cpu/avx512_bf16_rmsnorm_reduction.cpp:69-81. */
static float sum_lanes16(const float* lane) {
    float total[4];
    for (int j = 0; j < 4; ++j) {
        volatile float t = lane[j] + lane[j + 4];
        t = t + lane[j + 8];
        t = t + lane[j + 12];
        total[j] = t;
    }
    volatile float a = total[0] + total[2];
    volatile float b = total[1] + total[3];
    volatile float s = a + b;
    return s;
}

int iomo_rmsnorm(const iomo_view* x, const iomo_view* scale, const iomo_view* out,
                 float eps, int order) {
    geometry_t gx, gs, go;
    if (geometry_of(x, &gx) || geometry_of(scale, &gs) || geometry_of(out, &go)) return 1;
    if (x->dtype != out->dtype || x->dtype != scale->dtype) return 1;
    if (x->rank != out->rank || scale->rank != 2) return 1;
    for (uint32_t i = 0; i < x->rank; ++i) {
        if (x->dims[i] != out->dims[i]) return 1;
    }
    if (gs.rows != 1 || gs.columns != gx.columns) return 1;
    const format_t f = format_of(x->dtype);
    if (!f.bits || x->dtype == DT_F64) return 1; /* F64 carrier not restated */
    if (!(eps >= 0.0f) || isinf(eps)) return 1;
    const uint64_t features = gx.columns;
    const unsigned char* x_base = (const unsigned char*)x->base;
    const unsigned char* s_base = (const unsigned char*)scale->base;
    unsigned char* o_base = (unsigned char*)out->base;
    const uint64_t planes = leading_count(x);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t xp = view_plane(x, index);
        const uint64_t op = view_plane(out, index);
        for (uint64_t row = 0; row < gx.rows; ++row) {
            volatile float inverse = 0.0f;
            int reduced = 0;
            if (order == 0 && x->dtype == DT_BF16) {
                /* avx512_bf16_rmsnorm_reduce, avx512_bf16_rmsnorm_reduction.cpp:85-149 */
                float lane[16];
                for (int i = 0; i < 16; ++i) lane[i] = 0.0f;
                reduced = 1;
                for (uint64_t c = 0; c < features && reduced; ++c) {
                    const float v = (float)codec_decode(
                            load_bits(x_base, element_bit(x, &gx, xp, row, c), gx.bits), f);
                    if (isnan(v) || isinf(v)) {
                        reduced = 0;
                        break;
                    }
                    volatile float sq = v * v;
                    volatile float acc = lane[c % 16] + sq;
                    lane[c % 16] = acc;
                }
                if (reduced) {
                    const float sum = sum_lanes16(lane);
                    volatile float mean = sum / (float)features;
                    volatile float shifted = mean + eps;
                    volatile float root = sqrtf(shifted);
                    inverse = 1.0f / root;
                }
            }
            if (!reduced) {
                /* sequential recurrence, queue.cpp:1187-1196 */
                volatile float sum = 0.0f;
                for (uint64_t c = 0; c < features; ++c) {
                    const float v = (float)codec_decode(
                            load_bits(x_base, element_bit(x, &gx, xp, row, c), gx.bits), f);
                    volatile float sq = v * v;
                    sum = sum + sq;
                }
                volatile float mean = sum / (float)features;
                volatile float shifted = mean + eps;
                volatile float root = sqrtf(shifted);
                inverse = 1.0f / root;
            }
            /* second pass, queue.cpp:1225-1234 and encode_element :1117-1135 */
            for (uint64_t c = 0; c < features; ++c) {
                const float v = (float)codec_decode(
                        load_bits(x_base, element_bit(x, &gx, xp, row, c), gx.bits), f);
                const float w = (float)codec_decode(
                        load_bits(s_base,
                                  element_bit(scale, &gs, scale->plane_offset, 0, c), gs.bits),
                        f);
                volatile float normalized = v * inverse;
                volatile float scaled = normalized * w;
                float result = scaled;
                if (isnan(result)) result = fabsf(result);
                store_bits(o_base, element_bit(out, &go, op, row, c), go.bits,
                           codec_encode((long double)result, f));
            }
        }
    }
    return 0;
}

/* ---- copy: src/cpu/queue.cpp:2274-2303, src/device_ops_copy.cpp:17-52 ----- */

int iomo_copy(const iomo_view* source, const iomo_view* destination) {
    geometry_t gs, gd;
    if (geometry_of(source, &gs) || geometry_of(destination, &gd)) return 1;
    if (source->dtype != destination->dtype || source->rank != destination->rank) return 1;
    for (uint32_t i = 0; i < source->rank; ++i) {
        if (source->dims[i] != destination->dims[i]) return 1;
    }
    const uint64_t planes = leading_count(source);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t sp = view_plane(source, index);
        const uint64_t dp = view_plane(destination, index);
        for (uint64_t row = 0; row < gs.rows; ++row) {
            for (uint64_t column = 0; column < gs.columns; ++column) {
                const uint64_t value = load_bits(
                        (const unsigned char*)source->base,
                        element_bit(source, &gs, sp, row, column), gs.bits);
                store_bits((unsigned char*)destination->base,
                           element_bit(destination, &gd, dp, row, column), gd.bits, value);
            }
        }
    }
    return 0;
}

/* ---- cast (extension): codec decode then encode ------------------------- */

int iomo_cast(const iomo_view* source, const iomo_view* destination) {
    geometry_t gs, gd;
    if (geometry_of(source, &gs) || geometry_of(destination, &gd)) return 1;
    if (source->rank != destination->rank) return 1;
    for (uint32_t i = 0; i < source->rank; ++i) {
        if (source->dims[i] != destination->dims[i]) return 1;
    }
    if (!format_of(source->dtype).bits || !format_of(destination->dtype).bits) return 1;
    const uint64_t planes = leading_count(source);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t sp = view_plane(source, index);
        const uint64_t dp = view_plane(destination, index);
        for (uint64_t row = 0; row < gs.rows; ++row) {
            for (uint64_t column = 0; column < gs.columns; ++column) {
                const uint64_t raw = load_bits(
                        (const unsigned char*)source->base,
                        element_bit(source, &gs, sp, row, column), gs.bits);
                store_bits((unsigned char*)destination->base,
                           element_bit(destination, &gd, dp, row, column), gd.bits,
                           iomo_decode_encode(source->dtype, destination->dtype, raw));
            }
        }
    }
    return 0;
}

/* ---- SiLU: src/shared/scalar_silu.hpp:66-101 ------------------------------- */

/* scalar_silu_detail::evaluate on the FP32 carrier, the evaluation domain the CPU
 * backend selects for every leaf below F64 (src/cpu/queue.cpp:1770-1774,1863-1868;
 * the AVX-512 BF16 source runs the same FP32 operations, src/cpu/avx512_bf16_silu.cpp:147-176).
 * exp is the C library's expf, as std::exp(float) is there. Every operation is
 * rounded separately (this file is built with -ffp-contract=off). */
static float silu_evaluate_f32(float x) {
    if (isnan(x)) return NAN;
    if (isinf(x)) return signbit(x) ? -0.0f : INFINITY;
    if (x == 0.0f) return x;
    if (x >= 0.0f) {
        const float weight = expf(-x);
        const float denominator = 1.0f + weight;
        return x / denominator;
    }
    const float t = expf(x * 0.5f);
    const float first = x * t;
    const float numerator = first * t;
    const float square = t * t;
    const float denominator = 1.0f + square;
    return numerator / denominator;
}

/* The same evaluator on the FP64 carrier of the reference's GPU backends
 * (SiluFp64Traits, src/cuda/copy.cu:498-503). */
static double silu_evaluate_f64(double x) {
    if (isnan(x)) return NAN;
    if (isinf(x)) return signbit(x) ? -0.0 : INFINITY;
    if (x == 0.0) return x;
    if (x >= 0.0) {
        const double weight = exp(-x);
        const double denominator = 1.0 + weight;
        return x / denominator;
    }
    const double t = exp(x * 0.5);
    const double first = x * t;
    const double numerator = first * t;
    const double square = t * t;
    const double denominator = 1.0 + square;
    return numerator / denominator;
}

/* scalar_silu: decode the leaf, evaluate on the carrier, one RNE encode.
 * carrier 0: FP32 (CPU backend), 1: FP64 (GPU backends). */
uint64_t iomo_scalar_silu(uint32_t dtype, uint64_t raw, int carrier) {
    const format_t f = format_of(dtype);
    if (!f.bits) return 0;
    const long double value = codec_decode(raw, f);
    if (carrier == 0) {
        return codec_encode((long double)silu_evaluate_f32((float)value), f);
    }
    return codec_encode((long double)silu_evaluate_f64((double)value), f);
}

int iomo_silu(const iomo_view* x, const iomo_view* y, int carrier) {
    geometry_t gx, gy;
    if (geometry_of(x, &gx) || geometry_of(y, &gy)) return 1;
    if (x->dtype != y->dtype || x->rank != y->rank) return 1;
    for (uint32_t i = 0; i < x->rank; ++i) {
        if (x->dims[i] != y->dims[i]) return 1;
    }
    if (x->base == y->base) return 1;                /* src/device_ops_neural.cpp:362-368 */
    if (!format_of(x->dtype).bits) return 2;
    if (carrier != 0 && carrier != 1) return 1;
    const uint64_t planes = leading_count(x);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t xp = view_plane(x, index);
        const uint64_t yp = view_plane(y, index);
        for (uint64_t row = 0; row < gx.rows; ++row) {
            for (uint64_t column = 0; column < gx.columns; ++column) {
                const uint64_t raw = load_bits((const unsigned char*)x->base,
                                               element_bit(x, &gx, xp, row, column), gx.bits);
                store_bits((unsigned char*)y->base, element_bit(y, &gy, yp, row, column), gy.bits,
                           iomo_scalar_silu(x->dtype, raw, carrier));
            }
        }
    }
    return 0;
}

/* ---- RoPE: src/cpu/queue.cpp:1338-1592 ---------------------------------------- */

/* rope_angle on the FP32 carrier (src/cpu/queue.cpp:1356-1367): the exponent is
 * formed in FP64 and narrowed, powf / sinf / cosf are the C library's. */
void iomo_rope_angle(uint64_t column, uint64_t width, uint64_t position, float theta,
                     float* sine, float* cosine) {
    const float exponent = (float)((-2.0 * (double)column) / (double)width);
    const float frequency = powf(theta, exponent);
    const float angle = (float)position * frequency;
    *sine = sinf(angle);
    *cosine = cosf(angle);
}

/* Split-half rotary embedding of [..., H, R, W]: row r of every plane sits at
 * position a + r; columns c and c + W/2 form a pair. A row at position 0 is copied
 * raw (src/cpu/queue.cpp:1497-1522); every other pair is four separately rounded
 * FP32 products, one subtraction, one addition and one RNE encode each
 * (src/cpu/queue.cpp:1369-1411). Leaves below F64 only. */
int iomo_rope(const iomo_view* x, const iomo_view* out, uint64_t a, double theta) {
    geometry_t gx, go;
    if (geometry_of(x, &gx) || geometry_of(out, &go)) return 1;
    if (x->rank < 3 || x->rank != out->rank || x->dtype != out->dtype) return 1;
    for (uint32_t i = 0; i < x->rank; ++i) {
        if (x->dims[i] != out->dims[i]) return 1;
    }
    if (gx.columns % 2 != 0 || x->base == out->base) return 1;
    if (!(theta >= 1.0) || theta > 3.4028234663852886e38) return 1;
    const format_t f = format_of(x->dtype);
    if (!f.bits || f.bits > 32) return 2;
    const float narrowed = (float)theta;
    const uint64_t half = gx.columns / 2;
    const uint64_t planes = leading_count(x);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t xp = view_plane(x, index);
        const uint64_t op = view_plane(out, index);
        for (uint64_t row = 0; row < gx.rows; ++row) {
            const uint64_t position = a + row;
            if (position == 0) {
                for (uint64_t column = 0; column < gx.columns; ++column) {
                    store_bits((unsigned char*)out->base, element_bit(out, &go, op, row, column), go.bits,
                               load_bits((const unsigned char*)x->base,
                                         element_bit(x, &gx, xp, row, column), gx.bits));
                }
                continue;
            }
            for (uint64_t column = 0; column < half; ++column) {
                const float first = (float)codec_decode(
                        load_bits((const unsigned char*)x->base,
                                  element_bit(x, &gx, xp, row, column), gx.bits), f);
                const float second = (float)codec_decode(
                        load_bits((const unsigned char*)x->base,
                                  element_bit(x, &gx, xp, row, column + half), gx.bits), f);
                float sine, cosine;
                iomo_rope_angle(column, gx.columns, position, narrowed, &sine, &cosine);
                const volatile float first_product = first * cosine;
                const volatile float second_product = second * sine;
                const volatile float first_output = first_product - second_product;
                const volatile float second_cosine = second * cosine;
                const volatile float first_sine = first * sine;
                const volatile float second_output = second_cosine + first_sine;
                store_bits((unsigned char*)out->base, element_bit(out, &go, op, row, column), go.bits,
                           codec_encode((long double)first_output, f));
                store_bits((unsigned char*)out->base, element_bit(out, &go, op, row, column + half),
                           go.bits, codec_encode((long double)second_output, f));
            }
        }
    }
    return 0;
}

/* ---- embedding: src/cpu/queue.cpp:941-1038 -------------------------------- */

int iomo_embedding(const iomo_view* table, const iomo_view* indices,
                   const iomo_view* out, uint32_t* status) {
    geometry_t gt, gi, go;
    if (geometry_of(table, &gt) || geometry_of(indices, &gi) || geometry_of(out, &go)) return 1;
    if (table->rank != 2 || indices->rank != out->rank) return 1;
    if (table->dtype != out->dtype) return 1;
    const unsigned index_width = integer_width(indices->dtype);
    if (!index_width) return 1;
    if (gi.rows != 1 || gi.columns != go.rows || go.columns != gt.columns) return 1;
    for (uint32_t i = 0; i + 2 < out->rank; ++i) {
        if (indices->dims[i] != out->dims[i]) return 1;
    }
    const int is_signed = (indices->dtype % 2) == 1; /* I2,I4,...,I64 have odd ordinals */
    const uint64_t vocabulary = gt.rows;
    const uint64_t run = gi.columns;
    const uint64_t planes = leading_count(indices);
    *status = 0;
    /* validate every index first (queue.cpp:986-1010) */
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t ip = view_plane(indices, index);
        for (uint64_t r = 0; r < run; ++r) {
            const uint64_t raw = load_bits((const unsigned char*)indices->base,
                                           element_bit(indices, &gi, ip, 0, r), gi.bits);
            if (is_signed && ((raw >> (index_width - 1)) & 1u)) *status = 1;
            if (raw >= vocabulary) *status = 1;
        }
    }
    if (*status) return 0;
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t ip = view_plane(indices, index);
        const uint64_t op = view_plane(out, index);
        for (uint64_t r = 0; r < run; ++r) {
            const uint64_t id = load_bits((const unsigned char*)indices->base,
                                          element_bit(indices, &gi, ip, 0, r), gi.bits);
            for (uint64_t c = 0; c < gt.columns; ++c) {
                const uint64_t value = load_bits(
                        (const unsigned char*)table->base,
                        element_bit(table, &gt, table->plane_offset, id, c), gt.bits);
                store_bits((unsigned char*)out->base, element_bit(out, &go, op, r, c),
                           go.bits, value);
            }
        }
    }
    return 0;
}

/* ---- cache_append: src/cpu/queue.cpp:2227-2272,
 *      admission src/device_ops_cache_append.cpp:157-269 ------------------- */

int iomo_cache_append(const iomo_view* source, const iomo_view* destination, uint64_t a) {
    geometry_t gs, gd;
    if (geometry_of(source, &gs) || geometry_of(destination, &gd)) return 1;
    if (source->rank < 3 || source->rank != destination->rank) return 1;
    if (source->dtype != destination->dtype) return 1;
    for (uint32_t i = 0; i + 2 < source->rank; ++i) {
        if (source->dims[i] != destination->dims[i]) return 1;
    }
    if (gs.columns != gd.columns) return 1;
    if (a > gd.rows || gs.rows > gd.rows - a) return 1;
    const uint64_t planes = leading_count(source);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t sp = view_plane(source, index);
        const uint64_t dp = view_plane(destination, index);
        for (uint64_t row = 0; row < gs.rows; ++row) {
            for (uint64_t column = 0; column < gs.columns; ++column) {
                const uint64_t value = load_bits(
                        (const unsigned char*)source->base,
                        element_bit(source, &gs, sp, row, column), gs.bits);
                store_bits((unsigned char*)destination->base,
                           element_bit(destination, &gd, dp, a + row, column), gd.bits,
                           value);
            }
        }
    }
    return 0;
}

/* ---- sum of squares (extension): FP64 evaluation as the truth ------------ */

double iomo_sumsq(const iomo_view* x) {
    geometry_t g;
    if (geometry_of(x, &g)) return NAN;
    const format_t f = format_of(x->dtype);
    if (!f.bits) return NAN;
    double sum = 0.0;
    const uint64_t planes = leading_count(x);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t p = view_plane(x, index);
        for (uint64_t row = 0; row < g.rows; ++row) {
            for (uint64_t column = 0; column < g.columns; ++column) {
                const double v = (double)codec_decode(
                        load_bits((const unsigned char*)x->base,
                                  element_bit(x, &g, p, row, column), g.bits),
                        f);
                sum += v * v;
            }
        }
    }
    return sum;
}

/* ---- host transfers: src/cpu/tensor.cpp:78-163 --------------------------- */

int iomo_scatter(const iomo_view* destination, const void* logical) {
    geometry_t g;
    if (geometry_of(destination, &g)) return 1;
    const uint64_t planes = leading_count(destination);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t p = view_plane(destination, index);
        for (uint64_t row = 0; row < g.rows; ++row) {
            for (uint64_t column = 0; column < g.columns; ++column) {
                const uint64_t host_bit =
                        ((index * g.rows + row) * g.columns + column) * g.bits;
                store_bits((unsigned char*)destination->base,
                           element_bit(destination, &g, p, row, column), g.bits,
                           load_bits((const unsigned char*)logical, host_bit, g.bits));
            }
        }
    }
    return 0;
}

int iomo_gather(const iomo_view* source, void* logical) {
    geometry_t g;
    if (geometry_of(source, &g)) return 1;
    const uint64_t planes = leading_count(source);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t p = view_plane(source, index);
        for (uint64_t row = 0; row < g.rows; ++row) {
            for (uint64_t column = 0; column < g.columns; ++column) {
                const uint64_t host_bit =
                        ((index * g.rows + row) * g.columns + column) * g.bits;
                store_bits((unsigned char*)logical, host_bit, g.bits,
                           load_bits((const unsigned char*)source->base,
                                     element_bit(source, &g, p, row, column), g.bits));
            }
        }
    }
    return 0;
}

/* ---- attention stages without matrix products: src/cuda/sdpa_nonmatrix.cu:347-507 ---- */

static int sdpa_stages_ok(const iomo_sdpa_stages* q) {
    if (!q || !q->scores || !q->probability) return 0;
    if (!q->planes || !q->Hq || !q->Hkv || !q->R || !q->C || !q->D || !q->L) return 0;
    if (q->L > q->C || q->a >= q->C || q->R > q->C - q->a) return 0;
    return q->Hq % q->Hkv == 0;
}

static uint64_t sdpa_pad16(uint64_t v) { return (v + 15) / 16 * 16; }

static uint64_t sdpa_visible(const iomo_sdpa_stages* q, uint64_t row) {
    return q->L < q->a + row + 1 ? q->L : q->a + row + 1;
}

/* bf16_rne of src/cuda/sdpa_nonmatrix.cu:317-336. */
static uint16_t sdpa_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7f800000u) == 0x7f800000u) {
        return (bits & 0x007fffffu) == 0 ? (uint16_t)(bits >> 16) : (uint16_t)0x7fc0;
    }
    if ((bits & 0x7fffffffu) == 0) return 0;
    return (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

int iomo_sdpa_scale_mask(const iomo_sdpa_stages* q) {
    if (!sdpa_stages_ok(q)) return 1;
    const uint64_t Rp = sdpa_pad16(q->R), Lp = sdpa_pad16(q->L);
    const float scale = 1.0f / sqrtf((float)q->D);
    for (uint64_t head = 0; head < q->planes * q->Hq; ++head) {
        for (uint64_t row = 0; row < q->R; ++row) {
            float* cells = q->scores + (head * Rp + row) * Lp;
            const uint64_t visible = sdpa_visible(q, row);
            for (uint64_t token = 0; token < visible; ++token) {
                const volatile float scaled = cells[token] * scale;
                cells[token] = scaled == 0.0f ? 0.0f : scaled;
            }
        }
    }
    return 0;
}

int iomo_sdpa_softmax(const iomo_sdpa_stages* q) {
    if (!sdpa_stages_ok(q)) return 1;
    const uint64_t Rp = sdpa_pad16(q->R), Lp = sdpa_pad16(q->L);
    for (uint64_t head = 0; head < q->planes * q->Hq; ++head) {
        for (uint64_t row = 0; row < q->R; ++row) {
            const float* cells = q->scores + (head * Rp + row) * Lp;
            uint16_t* out = q->probability + (head * Rp + row) * Lp;
            const uint64_t visible = sdpa_visible(q, row);
            int has_nan = 0, all_negative = 1;
            uint64_t positive = 0;
            float maximum = -INFINITY;
            for (uint64_t token = 0; token < visible; ++token) {
                const float s = cells[token];
                if (isnan(s)) { has_nan = 1; continue; }
                if (isinf(s) && s > 0.0f) { ++positive; all_negative = 0; continue; }
                if (isinf(s)) continue;
                all_negative = 0;
                if (s > maximum) maximum = s;
            }
            if (has_nan || all_negative) {
                for (uint64_t token = 0; token < q->L; ++token) out[token] = token < visible ? 0x7fc0 : 0;
                continue;
            }
            if (positive) {
                const float share = 1.0f / (float)positive;
                for (uint64_t token = 0; token < q->L; ++token) {
                    const int hit = token < visible && isinf(cells[token]) && cells[token] > 0.0f;
                    out[token] = hit ? sdpa_bf16(share) : 0;
                }
                continue;
            }
            float sum = 0.0f;
            for (uint64_t token = 0; token < visible; ++token) {
                if (isinf(cells[token])) continue;
                const volatile float shifted = cells[token] - maximum;
                const volatile float next = sum + expf(shifted);
                sum = next;
            }
            for (uint64_t token = 0; token < q->L; ++token) {
                if (token >= visible || isinf(cells[token])) { out[token] = 0; continue; }
                const volatile float shifted = cells[token] - maximum;
                const volatile float quotient = expf(shifted) / sum;
                out[token] = sdpa_bf16(quotient);
            }
        }
    }
    return 0;
}

int iomo_sdpa_canonicalize_output(const iomo_view* out) {
    geometry_t g;
    if (geometry_of(out, &g) || out->dtype != 20) return 1;
    const uint64_t planes = leading_count(out);
    for (uint64_t index = 0; index < planes; ++index) {
        const uint64_t p = view_plane(out, index);
        for (uint64_t row = 0; row < g.rows; ++row) {
            for (uint64_t column = 0; column < g.columns; ++column) {
                const uint64_t bit = element_bit(out, &g, p, row, column);
                uint64_t bits = load_bits((const unsigned char*)out->base, bit, 16);
                if ((bits & 0x7fffu) == 0) bits = 0;
                else if ((bits & 0x7f80u) == 0x7f80u && (bits & 0x007fu) != 0) bits = 0x7fc0u;
                store_bits((unsigned char*)out->base, bit, 16, bits);
            }
        }
    }
    return 0;
}
