// C++ host side of the B200 backend: an iom::Device whose tensors live in the
// standard tiled layout inside one device arena and whose operation queue
// launches the kernels of libiom_b200.so (include/iom_b200.h).
//
// It plugs into the reference's own headers (include/iom/device.hpp,
// include/iom/iom.hpp): build it with the reference checkout on the include
// path. The factory mirrors make_cuda_device (include/iom/cuda/device.hpp:22-24).
#pragma once

#include <cstdint>
#include <memory>

#include "iom/device.hpp"
#include "iom/iom.hpp"

namespace iom {

// Rejects a zero or non-multiple-of-32 arena with std::invalid_argument, an
// unknown ordinal with std::invalid_argument, a failed reservation with
// std::bad_alloc. Reports BackendKind::CUDA (the enum has no spare value).
[[nodiscard]] std::unique_ptr<Device> make_b200_device(
        std::uint32_t ordinal, DeviceMemoryConfig memory_config,
        QueueConfig queue_config = {});

namespace b200 {

// Extension outside the DeviceOps facade: residual ADD fused into the
// following RMSNorm (sum = x + residual is stored; out = rmsnorm(sum, scale)).
// `queue` must have been created by a device from make_b200_device. Returns
// an oid like the facade operations do.
oid add_rmsnorm(DeviceOps& queue, const TensorView& x, const TensorView& residual,
                const TensorView& scale, TensorView& sum, TensorView& out, float eps);

// Extension outside the DeviceOps facade: out = silu(x) * up in one pass, the
// decoder MLP's SiLU(gate) followed by the multiply with the up projection.
// `activated` (may be null) receives silu(x). Results equal silu then mul.
oid silu_mul(DeviceOps& queue, const TensorView& x, const TensorView& up, TensorView* activated,
             TensorView& out);

// BF16 <-> F32 conversion between views of identical logical shape (codec decode /
// encode: exact widening, RNE narrowing, canonical NaN).
oid cast(DeviceOps& queue, const TensorView& source, TensorView& destination);

// cache_append with one row offset per index of the first leading axis (a decode step's
// K or V of every sequence in one launch). `positions` (dims[0] values) and `status`
// (one word: reset to 0, set to 1 when some offset overruns its cache, that sequence
// being skipped) are device addresses the caller owns until the token completes.
oid cache_append_batched(DeviceOps& queue, const TensorView& source, TensorView& destination,
                         const std::uint32_t* positions, std::uint32_t* status);

// Whole-view FP32 sum of squares with a launch-independent order into the device float at
// `result`; `scratch` is sumsq_scratch_bytes() bytes of device memory.
oid sumsq(DeviceOps& queue, const TensorView& x, void* scratch, float* result);
[[nodiscard]] std::size_t sumsq_scratch_bytes();

// The attention stages that are not matrix products, on the two workspace segments of the
// reference's CUDA backend (src/cuda/sdpa_nonmatrix_request.hpp:22-49): FP32 scores and BF16
// probabilities, both [planes, Hq, pad16(R), pad16(L)], device pointers aligned to 32 bytes.
// They replace launch_sdpa_scale_mask / launch_sdpa_softmax / launch_sdpa_canonicalize_output
// (src/cuda/sdpa_nonmatrix.hpp:15-28); sdpa_scale_mask_softmax does the first two in one pass
// and stores the scaled scores only when asked to.
struct SdpaStages {
    float* scores = nullptr;
    void* probability = nullptr;
    std::uint64_t planes = 0, Hq = 0, Hkv = 0, R = 0, C = 0, D = 0, a = 0, L = 0;
};
oid sdpa_scale_mask(DeviceOps& queue, const SdpaStages& stages);
oid sdpa_softmax(DeviceOps& queue, const SdpaStages& stages);
oid sdpa_scale_mask_softmax(DeviceOps& queue, const SdpaStages& stages, bool keep_scores);
oid sdpa_canonicalize_output(DeviceOps& queue, TensorView& out);

}  // namespace b200
}  // namespace iom
