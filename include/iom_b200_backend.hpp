// C++ host side of the B200 backend: an iom::Device whose tensors live in the
// standard tiled layout inside one device arena and whose operation queue
// launches the kernels of libiom_b200.so (include/iom_b200.h).
//
// It plugs into the reference's own headers (include/iom/device.hpp,
// include/iom/iom.hpp): build it with the reference checkout on the include
// path. The factory mirrors make_cuda_device (include/iom/cuda/device.hpp:22-24).
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>

#include "iom/device.hpp"
#include "iom/iom.hpp"

namespace iom {

namespace b200 {
// Set-up choices beyond the reference's DeviceMemoryConfig / QueueConfig. Everything the
// device will ever allocate natively is reserved at construction (the contract allows no
// native allocation afterwards, docs/BACKEND_CONTRACT/memory-admission-and-workspace-contract.md:17-24):
// the tensor arena, and one region for rotary (cos, sin) tables. A RoPE request whose
// table no longer fits the region is refused with ResourceExhausted.
struct Options {
    std::size_t rotary_table_bytes = 8u << 20;   // 0 = RoPE reports ResourceExhausted
};
}  // namespace b200

// Rejects a zero or non-multiple-of-32 arena with std::invalid_argument, an
// unknown ordinal with std::invalid_argument, a failed reservation with
// std::bad_alloc. Reports BackendKind::CUDA (the enum has no spare value).
// Native allocations: the tensor arena and the rotary region (two cudaMalloc calls),
// at construction only.
[[nodiscard]] std::unique_ptr<Device> make_b200_device(
        std::uint32_t ordinal, DeviceMemoryConfig memory_config,
        QueueConfig queue_config = {}, b200::Options options = {});

namespace b200 {

// Every extension below takes a queue created by a device from make_b200_device (any
// other queue: InvalidArgument) and returns an oid like the facade operations do. Each
// registers the owners of its views, and leases the workspace ranges it is given, until
// the token's completion is proven — destroying an operand before `wait` parks its
// storage instead of recycling it, as for the facade operations.

// Residual ADD fused into the following RMSNorm (sum = x + residual is stored;
// out = rmsnorm(sum, scale)). Results equal add then rmsnorm bit for bit.
oid add_rmsnorm(DeviceOps& queue, const TensorView& x, const TensorView& residual,
                const TensorView& scale, TensorView& sum, TensorView& out, float eps);

// out = silu(x) * up in one pass, the decoder MLP's SiLU(gate) followed by the multiply
// with the up projection. `activated` (may be null) receives silu(x).
oid silu_mul(DeviceOps& queue, const TensorView& x, const TensorView& up, TensorView* activated,
             TensorView& out);

// BF16 <-> F32 conversion between views of identical logical shape (codec decode /
// encode: exact widening, RNE narrowing, canonical NaN).
oid cast(DeviceOps& queue, const TensorView& source, TensorView& destination);

// cache_append with one row offset per index of the first leading axis (a decode step's
// K or V of every sequence in one launch). `control` is a workspace range of at least
// batched_control_bytes(dims[0]) bytes of this device: its first u32 is the status word
// (reset to 0 by the call, 1 when some offset overruns its cache, that sequence being
// skipped), the u32 row offsets start at byte 32. The caller fills the offsets (device
// memory) before the call and reads the status after the token completes. The range is
// registered like an operand, not leased exclusively: several appends in flight on one
// queue (K and V of every layer of a step) may name the same offsets.
oid cache_append_batched(DeviceOps& queue, const TensorView& source, TensorView& destination,
                         RawWorkspaceView control);
[[nodiscard]] std::size_t batched_control_bytes(std::size_t sequences);

// Whole-view FP32 sum of squares with a launch-independent order. `workspace` is a range
// of at least sumsq_workspace_bytes() bytes of this device; the FP32 result lands in its
// first four bytes (the rest is scratch).
oid sumsq(DeviceOps& queue, const TensorView& x, RawWorkspaceView workspace);
[[nodiscard]] std::size_t sumsq_workspace_bytes();

// The attention stages that are not matrix products, on the two workspace segments of the
// reference's CUDA backend (src/cuda/sdpa_nonmatrix_request.hpp:22-49): FP32 scores and BF16
// probabilities, both [planes, Hq, pad16(R), pad16(L)], device pointers aligned to 32 bytes
// inside `workspace` (leased for the call). They replace launch_sdpa_scale_mask /
// launch_sdpa_softmax / launch_sdpa_canonicalize_output (src/cuda/sdpa_nonmatrix.hpp:15-28);
// sdpa_scale_mask_softmax does the first two in one pass and stores the scaled scores only
// when asked to.
struct SdpaStages {
    float* scores = nullptr;
    void* probability = nullptr;
    std::uint64_t planes = 0, Hq = 0, Hkv = 0, R = 0, C = 0, D = 0, a = 0, L = 0;
};
oid sdpa_scale_mask(DeviceOps& queue, const SdpaStages& stages, RawWorkspaceView workspace);
oid sdpa_softmax(DeviceOps& queue, const SdpaStages& stages, RawWorkspaceView workspace);
oid sdpa_scale_mask_softmax(DeviceOps& queue, const SdpaStages& stages, bool keep_scores,
                            RawWorkspaceView workspace);
oid sdpa_canonicalize_output(DeviceOps& queue, TensorView& out);

// ---- launch-bound sequences ---------------------------------------------------------
// A fixed sequence of operations (a decode step: docs/BACKEND_CONTRACT/
// tinyllama-forward-layout-workspace-and-execution.md:299-316 fixes its schedule) can be
// recorded once and replayed as one submission. Between capture_begin and capture_end the
// queue's operations are validated and admitted as usual but only recorded; their tokens
// complete at once and mean nothing. `replay` submits the whole recording as one
// operation with one token; embedding status words of the recording are checked when that
// token completes. The recording holds device addresses: every tensor and workspace it
// names must outlive it. Issue the sequence once eagerly before recording it.
class CapturedSequence;
void capture_begin(DeviceOps& queue);
[[nodiscard]] std::shared_ptr<CapturedSequence> capture_end(DeviceOps& queue);
oid replay(DeviceOps& queue, const std::shared_ptr<CapturedSequence>& sequence);

// The queue's CUDA stream (a cudaStream_t), for callers that time with CUDA events.
[[nodiscard]] void* native_stream(DeviceOps& queue);

// ---- host-side failure injection (tests) ---------------------------------------------
// The points of the reference's CUDA policy (src/cuda/copy.hpp:41-60) that exist here;
// each substitutes an error code at a host call site, no device is ever faulted.
//   launch                 the next kernel launch reports a failure before launching
//   embedding_status_copy  the next status-word copy of an embedding fails
//   event_record           the next two event records and the next stream drain fail:
//                          completion cannot be proven, so the operation's owners are
//                          invalidated, its lease and its event are quarantined
//   stream_synchronize     the next stream drain fails
//   registration, outcome_insertion
//                          the next submission fails before acceptance (ResourceExhausted)
enum class SubmissionFault {
    none, launch, embedding_status_copy, event_record, stream_synchronize, registration,
    outcome_insertion
};
void inject_submission_fault_for_testing(SubmissionFault fault) noexcept;
// Events of the queue that are quarantined (never reused) after an unproven completion.
[[nodiscard]] std::size_t quarantined_event_count(DeviceOps& queue);

}  // namespace b200
}  // namespace iom
