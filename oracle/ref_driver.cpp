// TEST INFRASTRUCTURE — not part of the product.
//
// C-ABI shim over the *unmodified* reference CPU backend (rlewczuk/iom). It is
// compiled together with the reference's own sources where they lie (see the
// Makefile beside this file) into oracle/_ref/libiomref_{portable,avx512}.so.
// The shim only exposes the reference's public API (Device, Tensor,
// TensorView transforms, DeviceOps facades, wait) to ctypes so that tests can
//   * pin the plain-C restatement in iom_oracle.c against the real reference,
//   * generate the golden fixtures committed under tests/golden/,
//   * time the reference CPU backend as the reported CPU baseline.
// Nothing in the product library links or loads this file.
//
// Reference interfaces wrapped here:
//   make_cpu_device                 include/iom/cpu/device.hpp:19-20
//   Device::create_tensor/create_ops include/iom/device.hpp:86-99
//   TensorView transforms/transfers include/iom/tensor.hpp:322-342
//   DeviceOps::{copy,add,mul,sub,div,rmsnorm,embedding,cache_append,wait}
//                                   include/iom/iom.hpp:121-323

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <new>
#include <span>
#include <stdexcept>
#include <string>
#include <vector>

#include "iom/cpu/device.hpp"
#include "iom/iom.hpp"
#include "iom/tensor.hpp"

// With IOMREF_WITH_B200 the same shim can also create the B200 backend
// (iom_b200/backend/b200_backend.cpp) behind the reference's own DeviceOps
// facade, so one test can drive candidate and reference through identical calls.
#ifdef IOMREF_WITH_B200
#include <cuda_runtime_api.h>

#include "iom_b200_backend.hpp"
#endif

namespace iom::cpu_detail {
// src/cpu/avx512_bf16.hpp: true when this build and this CPU may enter the
// isolated AVX-512 BF16 workers.
bool avx512_bf16_available() noexcept;
}  // namespace iom::cpu_detail

namespace {

thread_local std::string g_last_error;

class AlignedHostAllocator final : public iom::Allocator {
public:
    void* alloc(std::size_t size) override {
        return ::operator new(size, std::align_val_t(64));
    }
    void free(void* buffer) override {
        ::operator delete(buffer, std::align_val_t(64));
    }
    void reset() override {}
};

struct DeviceBox {
    AlignedHostAllocator allocator;
    std::unique_ptr<iom::Device> device;
    bool accelerator = false;
    // Workspaces handed to operations stay alive until the device goes away.
    std::vector<std::unique_ptr<iom::RawWorkspace>> workspaces;

    ~DeviceBox() { workspaces.clear(); }

    iom::RawWorkspaceView workspace(const iom::WorkspaceRequirements& need) {
        if (need.bytes == 0) return {};
        workspaces.push_back(device->create_workspace(need.bytes));
        return workspaces.back()->view();
    }
};

struct TensorBox {
    std::unique_ptr<iom::Tensor> tensor;
    DeviceBox* device = nullptr;
};

struct ViewBox {
    iom::TensorView view;
    DeviceBox* device = nullptr;
};

struct QueueBox {
    std::unique_ptr<iom::DeviceOps> ops;
    DeviceBox* device = nullptr;
};

// Exception class → small positive code (0 is success).
int classify(std::exception_ptr failure) {
    try {
        std::rethrow_exception(failure);
    } catch (const std::invalid_argument& e) {
        g_last_error = e.what();
        return 1;
    } catch (const std::out_of_range& e) {
        g_last_error = e.what();
        return 2;
    } catch (const std::overflow_error& e) {
        g_last_error = e.what();
        return 3;
    } catch (const std::bad_alloc& e) {
        g_last_error = e.what();
        return 4;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return 5;
    } catch (...) {
        g_last_error = "unknown exception";
        return 6;
    }
}

template <typename Body>
void* guarded_pointer(Body&& body) {
    try {
        return body();
    } catch (...) {
        (void)classify(std::current_exception());
        return nullptr;
    }
}

template <typename Body>
int guarded_status(Body&& body) {
    try {
        body();
        return 0;
    } catch (...) {
        return classify(std::current_exception());
    }
}

iom::TensorView& view_of(void* handle) {
    return static_cast<ViewBox*>(handle)->view;
}

iom::DeviceOps& ops_of(void* handle) {
    return *static_cast<QueueBox*>(handle)->ops;
}

}  // namespace

extern "C" {

const char* iomref_last_error() { return g_last_error.c_str(); }

int iomref_avx512_bf16_active() {
    return iom::cpu_detail::avx512_bf16_available() ? 1 : 0;
}

void* iomref_device_create() {
    return guarded_pointer([]() -> void* {
        auto box = std::make_unique<DeviceBox>();
        box->device = iom::make_cpu_device(box->allocator);
        return box.release();
    });
}

void iomref_device_destroy(void* device) {
    delete static_cast<DeviceBox*>(device);
}

void* iomref_tensor_create(
        void* device, const std::uint64_t* dims, std::uint32_t rank,
        std::uint32_t data_type) {
    return guarded_pointer([&]() -> void* {
        std::vector<std::size_t> shape(dims, dims + rank);
        iom::TensorSpec spec{
                iom::TensorShape{std::move(shape)},
                static_cast<iom::DataType>(data_type)};
        auto box = std::make_unique<TensorBox>();
        box->device = static_cast<DeviceBox*>(device);
        box->tensor = box->device->device->create_tensor(spec);
        return box.release();
    });
}

void iomref_tensor_destroy(void* tensor) {
    delete static_cast<TensorBox*>(tensor);
}

// Raw tiled owner storage of a CPU tensor (src/cpu/tensor.cpp:36-76 reports the
// host buffer as the native handle).
void* iomref_tensor_storage(void* tensor) {
    return static_cast<TensorBox*>(tensor)->tensor->view().native_handle();
}

std::uint64_t iomref_tensor_storage_nbytes(void* tensor) {
    return static_cast<TensorBox*>(tensor)
            ->tensor->view().spec().tiled_storage_nbytes();
}

void* iomref_view_full(void* tensor) {
    return guarded_pointer([&]() -> void* {
        auto* owner = static_cast<TensorBox*>(tensor);
        return new ViewBox{owner->tensor->view(), owner->device};
    });
}

void* iomref_view_slice(
        void* view, std::uint64_t dim, std::uint64_t first,
        std::uint64_t count, std::uint64_t step) {
    return guarded_pointer([&]() -> void* {
        return new ViewBox{view_of(view).slice(dim, first, count, step), static_cast<ViewBox*>(view)->device};
    });
}

void* iomref_view_select(void* view, std::uint64_t dim, std::uint64_t index) {
    return guarded_pointer([&]() -> void* {
        return new ViewBox{view_of(view).select(dim, index), static_cast<ViewBox*>(view)->device};
    });
}

void* iomref_view_permute(
        void* view, const std::uint64_t* order, std::uint32_t count) {
    return guarded_pointer([&]() -> void* {
        std::vector<std::size_t> leading(order, order + count);
        return new ViewBox{view_of(view).permute(leading), static_cast<ViewBox*>(view)->device};
    });
}

void* iomref_view_reshape_leading(
        void* view, const std::uint64_t* dims, std::uint32_t count) {
    return guarded_pointer([&]() -> void* {
        std::vector<std::size_t> leading(dims, dims + count);
        return new ViewBox{view_of(view).reshape_leading(leading), static_cast<ViewBox*>(view)->device};
    });
}

void iomref_view_destroy(void* view) { delete static_cast<ViewBox*>(view); }

// Reports the metadata an operation snapshots from a view: full logical
// shape, leaf type, plane offset and leading plane strides (whole planes).
int iomref_view_describe(
        void* view, std::uint32_t* rank, std::uint64_t* dims,
        std::uint64_t* plane_offset, std::uint64_t* plane_strides,
        std::uint32_t* data_type) {
    return guarded_status([&] {
        const iom::TensorView& v = view_of(view);
        const auto shape = v.spec().shape.dimensions();
        *rank = static_cast<std::uint32_t>(shape.size());
        for (std::size_t i = 0; i < shape.size(); ++i) dims[i] = shape[i];
        *plane_offset = v.plane_offset();
        const auto strides = v.plane_strides();
        for (std::size_t i = 0; i < strides.size(); ++i) {
            plane_strides[i] = strides[i];
        }
        *data_type = static_cast<std::uint32_t>(v.spec().data_type);
    });
}

std::uint64_t iomref_view_logical_nbytes(void* view) {
    try {
        return view_of(view).spec().logical_nbytes();
    } catch (...) {
        (void)classify(std::current_exception());
        return 0;
    }
}

int iomref_view_from_host(void* view, const void* bytes, std::uint64_t count) {
    return guarded_status([&] {
        iom::TensorView& target = view_of(view);
        target.copy_from_host(
                std::span<const std::byte>(static_cast<const std::byte*>(bytes), count),
                static_cast<ViewBox*>(view)->device->workspace(
                        target.copy_from_host_workspace_requirements()));
    });
}

int iomref_view_to_host(void* view, void* bytes, std::uint64_t count) {
    return guarded_status([&] {
        iom::TensorView& source = view_of(view);
        source.copy_to_host(
                std::span<std::byte>(static_cast<std::byte*>(bytes), count),
                static_cast<ViewBox*>(view)->device->workspace(
                        source.copy_to_host_workspace_requirements()));
    });
}

void* iomref_queue_create(void* device) {
    return guarded_pointer([&]() -> void* {
        auto box = std::make_unique<QueueBox>();
        box->device = static_cast<DeviceBox*>(device);
        box->ops = box->device->device->create_ops();
        return box.release();
    });
}

void iomref_queue_destroy(void* queue) { delete static_cast<QueueBox*>(queue); }

// operation: 0 add, 1 mul, 2 sub, 3 div. Returns the facade's oid unchanged
// (negative = synchronous OidError, positive = accepted token).
std::int64_t iomref_binary(
        void* queue, int operation, void* lhs, void* rhs, void* out) {
    iom::DeviceOps& ops = ops_of(queue);
    switch (operation) {
        case 0: return ops.add(view_of(lhs), view_of(rhs), view_of(out));
        case 1: return ops.mul(view_of(lhs), view_of(rhs), view_of(out));
        case 2: return ops.sub(view_of(lhs), view_of(rhs), view_of(out));
        case 3: return ops.div(view_of(lhs), view_of(rhs), view_of(out));
        default: return -1;
    }
}

std::int64_t iomref_rmsnorm(
        void* queue, void* x, void* scale, void* out, float epsilon) {
    return ops_of(queue).rmsnorm(
            view_of(x), view_of(scale), view_of(out), epsilon);
}

std::int64_t iomref_silu(void* queue, void* x, void* y) {
    return ops_of(queue).silu(view_of(x), view_of(y));
}

std::int64_t iomref_rope(void* queue, void* x, void* out, std::uint64_t a, double theta) {
    return ops_of(queue).rope(view_of(x), view_of(out), a, theta);
}

std::int64_t iomref_copy(void* queue, void* source, void* destination) {
    return ops_of(queue).copy(view_of(source), view_of(destination));
}

std::int64_t iomref_embedding(
        void* queue, void* table, void* indices, void* out) {
    auto* box = static_cast<QueueBox*>(queue);
    try {
        const iom::WorkspaceRequirements need = box->ops->embedding_workspace_requirements(
                view_of(table), view_of(indices), view_of(out));
        return box->ops->embedding(view_of(table), view_of(indices), view_of(out),
                                   box->device->workspace(need));
    } catch (...) {
        // The query throws what the facade would map; let the facade report it.
        return box->ops->embedding(view_of(table), view_of(indices), view_of(out));
    }
}

std::int64_t iomref_cache_append(
        void* queue, void* source, void* destination, std::uint64_t a) {
    return ops_of(queue).cache_append(
            view_of(source), view_of(destination), a);
}

// 0 when the accepted work completed; otherwise the class of the retained or
// validation failure `wait` rethrew (1 invalid_argument, 3 overflow, ...).
int iomref_wait(void* queue, std::int64_t token) {
    return guarded_status([&] { ops_of(queue).wait(token); });
}

#ifdef IOMREF_WITH_B200
void* iomref_device_create_b200(std::uint32_t ordinal, std::uint64_t arena_bytes) {
    return guarded_pointer([&]() -> void* {
        auto box = std::make_unique<DeviceBox>();
        box->accelerator = true;
        box->device = iom::make_b200_device(ordinal, iom::DeviceMemoryConfig{arena_bytes});
        return box.release();
    });
}

// Whole-owner physical storage transfers through an independent native path
// (plain cudaMemcpy on the default stream), as the reference's CUDA storage
// oracle does (test/cuda/test_cuda_conformance.cpp:180-208).
int iomref_tensor_upload(void* tensor, const void* bytes, std::uint64_t count) {
    auto* box = static_cast<TensorBox*>(tensor);
    if (cudaMemcpy(box->tensor->view().native_handle(), bytes, count, cudaMemcpyHostToDevice)
            != cudaSuccess) {
        g_last_error = "cudaMemcpy H2D failed";
        return 5;
    }
    return 0;
}

int iomref_tensor_download(void* tensor, void* bytes, std::uint64_t count) {
    auto* box = static_cast<TensorBox*>(tensor);
    if (cudaDeviceSynchronize() != cudaSuccess
            || cudaMemcpy(bytes, box->tensor->view().native_handle(), count,
                          cudaMemcpyDeviceToHost) != cudaSuccess) {
        g_last_error = "cudaMemcpy D2H failed";
        return 5;
    }
    return 0;
}

std::int64_t iomref_add_rmsnorm(void* queue, void* x, void* residual, void* scale, void* sum,
                                void* out, float epsilon) {
    return iom::b200::add_rmsnorm(ops_of(queue), view_of(x), view_of(residual), view_of(scale),
                                  view_of(sum), view_of(out), epsilon);
}

std::int64_t iomref_silu_mul(void* queue, void* x, void* up, void* activated, void* out) {
    return iom::b200::silu_mul(ops_of(queue), view_of(x), view_of(up),
                               activated != nullptr ? &view_of(activated) : nullptr, view_of(out));
}

std::int64_t iomref_cast(void* queue, void* source, void* destination) {
    return iom::b200::cast(ops_of(queue), view_of(source), view_of(destination));
}

// positions: host array of `count` row offsets, staged into a control workspace of the
// device (status word first, offsets from byte 32). Returns the token; *status_out receives
// the status word after completion.
std::int64_t iomref_cache_append_batched(void* queue, void* source, void* destination,
                                         const std::uint32_t* positions, std::uint32_t count,
                                         std::uint32_t* status_out) {
    auto* box = static_cast<QueueBox*>(queue);
    std::unique_ptr<iom::RawWorkspace> control;
    try {
        control = box->device->device->create_workspace(iom::b200::batched_control_bytes(count));
    } catch (...) {
        return -4;
    }
    auto* words = static_cast<std::uint32_t*>(
            iom::detail::WorkspaceValidation::address(control->view()));
    cudaMemcpy(words + 8, positions, count * sizeof(std::uint32_t), cudaMemcpyHostToDevice);
    const std::int64_t token = iom::b200::cache_append_batched(
            ops_of(queue), view_of(source), view_of(destination), control->view());
    if (token > 0) {
        try {
            ops_of(queue).wait(token);
        } catch (...) {
        }
        cudaMemcpy(status_out, words, sizeof(std::uint32_t), cudaMemcpyDeviceToHost);
    }
    return token;
}

std::int64_t iomref_sumsq(void* queue, void* x, float* value_out) {
    auto* box = static_cast<QueueBox*>(queue);
    std::unique_ptr<iom::RawWorkspace> workspace;
    try {
        workspace = box->device->device->create_workspace(iom::b200::sumsq_workspace_bytes());
    } catch (...) {
        return -4;
    }
    const std::int64_t token = iom::b200::sumsq(ops_of(queue), view_of(x), workspace->view());
    if (token > 0) {
        try {
            ops_of(queue).wait(token);
        } catch (...) {
        }
        cudaMemcpy(value_out, iom::detail::WorkspaceValidation::address(workspace->view()),
                   sizeof(float), cudaMemcpyDeviceToHost);
    }
    return token;
}

// A workspace of the device for callers that place buffers themselves (the attention
// stage segments); returns the owner and writes its device address.
void* iomref_workspace_create(void* device, std::uint64_t bytes, void** address_out) {
    return guarded_pointer([&]() -> void* {
        auto* box = static_cast<DeviceBox*>(device);
        box->workspaces.push_back(box->device->create_workspace(bytes));
        *address_out = iom::detail::WorkspaceValidation::address(box->workspaces.back()->view());
        return box->workspaces.back().get();
    });
}

// Plain copies between host memory and a device address (synchronous).
int iomref_memcpy_b200(void* destination, const void* source, std::uint64_t bytes, int to_device) {
    if (cudaDeviceSynchronize() != cudaSuccess
            || cudaMemcpy(destination, source, bytes,
                          to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost) != cudaSuccess) {
        g_last_error = "cudaMemcpy failed";
        return 5;
    }
    return 0;
}

// stage 0..3 as B200Queue::sdpa_stage, 4 = canonicalise `out`; scores and probability are
// device addresses inside `workspace` (an owner from iomref_workspace_create).
std::int64_t iomref_sdpa_stage_b200(void* queue, int stage, void* scores, void* probability,
                                    const std::uint64_t* geometry, void* out, void* workspace) {
    std::int64_t token;
    if (stage == 4) {
        token = iom::b200::sdpa_canonicalize_output(ops_of(queue), view_of(out));
    } else {
        iom::b200::SdpaStages s;
        s.scores = static_cast<float*>(scores);
        s.probability = probability;
        s.planes = geometry[0]; s.Hq = geometry[1]; s.Hkv = geometry[2]; s.R = geometry[3];
        s.C = geometry[4]; s.D = geometry[5]; s.a = geometry[6]; s.L = geometry[7];
        const iom::RawWorkspaceView range = static_cast<iom::RawWorkspace*>(workspace)->view();
        if (stage == 0) token = iom::b200::sdpa_scale_mask(ops_of(queue), s, range);
        else if (stage == 1) token = iom::b200::sdpa_softmax(ops_of(queue), s, range);
        else token = iom::b200::sdpa_scale_mask_softmax(ops_of(queue), s, stage == 3, range);
    }
    if (token > 0) {
        try {
            ops_of(queue).wait(token);
        } catch (...) {
            return -5;
        }
    }
    return token;
}

// Host-side failure injection of the B200 backend: the ordinal of b200::SubmissionFault.
void iomref_inject_fault_b200(int fault) {
    iom::b200::inject_submission_fault_for_testing(static_cast<iom::b200::SubmissionFault>(fault));
}

std::uint64_t iomref_quarantined_events_b200(void* queue) {
    return iom::b200::quarantined_event_count(ops_of(queue));
}

void iomref_tensor_destroy_b200(void* tensor) { delete static_cast<TensorBox*>(tensor); }

// Recording and replay of a fixed sequence.
int iomref_capture_begin_b200(void* queue) {
    return guarded_status([&] { iom::b200::capture_begin(ops_of(queue)); });
}

void* iomref_capture_end_b200(void* queue) {
    return guarded_pointer([&]() -> void* {
        return new std::shared_ptr<iom::b200::CapturedSequence>(
                iom::b200::capture_end(ops_of(queue)));
    });
}

std::int64_t iomref_replay_b200(void* queue, void* recording) {
    return iom::b200::replay(
            ops_of(queue), *static_cast<std::shared_ptr<iom::b200::CapturedSequence>*>(recording));
}

void iomref_recording_destroy_b200(void* recording) {
    delete static_cast<std::shared_ptr<iom::b200::CapturedSequence>*>(recording);
}
#endif

}  // extern "C"
