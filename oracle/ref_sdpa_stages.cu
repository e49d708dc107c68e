// TEST INFRASTRUCTURE — not part of the product.
//
// C shim over the reference's own CUDA attention stage kernels
// (src/cuda/sdpa_nonmatrix.cu, compiled unmodified from the reference checkout by the
// Makefile beside this file into oracle/_ref/libiomref_sdpa_stages.so). The GPU parity
// tests run these launches next to the product's on the same device buffers and compare
// bits. Stage: 0 scale/mask, 1 softmax, 2 canonicalise output. Returns 0, or 1 when the
// reference threw (the text is kept for iomref_sdpa_error).
#include <cuda_runtime_api.h>

#include <cstdint>
#include <exception>
#include <string>

#include "cuda/sdpa_nonmatrix.hpp"

namespace {
thread_local std::string g_error;
}

extern "C" const char* iomref_sdpa_error() { return g_error.c_str(); }

extern "C" int iomref_sdpa_stage(
        int stage, float* scores, void* probability, void* output, std::uint64_t output_bytes,
        std::uint64_t output_plane_offset, const std::uint64_t* output_plane_strides,
        std::uint32_t leading_rank, const std::uint64_t* leading_dimensions,
        std::uint64_t Hq, std::uint64_t Hkv, std::uint64_t R, std::uint64_t C, std::uint64_t D,
        std::uint64_t a, std::uint64_t L, void* stream) {
    iom::cuda_detail::SdpaNonmatrixRequest request;
    request.scores = scores;
    request.probability = static_cast<unsigned char*>(probability);
    request.output.data = static_cast<unsigned char*>(output);
    request.output.storage_bytes = output_bytes;
    request.output.plane_offset = output_plane_offset;
    request.leading_rank = leading_rank;
    request.planes = 1;
    for (std::uint32_t axis = 0; axis < leading_rank; ++axis) {
        request.leading_dimensions[axis] = leading_dimensions[axis];
        request.output.plane_strides[axis] = output_plane_strides[axis];
        request.planes *= leading_dimensions[axis];
    }
    request.Hq = Hq;
    request.Hkv = Hkv;
    request.R = R;
    request.C = C;
    request.D = D;
    request.a = a;
    request.L = L;
    request.grouping = Hkv == 0 ? 0 : Hq / Hkv;
    request.Rp = (R + 15) / 16 * 16;
    request.Lp = (L + 15) / 16 * 16;
    int device = 0;
    (void)cudaGetDevice(&device);
    request.device_ordinal = static_cast<std::uint32_t>(device);
    try {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        if (stage == 0) iom::cuda_detail::launch_sdpa_scale_mask(s, request);
        else if (stage == 1) iom::cuda_detail::launch_sdpa_softmax(s, request);
        else iom::cuda_detail::launch_sdpa_canonicalize_output(s, request);
    } catch (const std::exception& error) {
        g_error = error.what();
        return 1;
    }
    return 0;
}
