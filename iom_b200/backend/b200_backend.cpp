// B200 backend for IOM's backend contract: Device / Tensor / RawWorkspace /
// DeviceOps subclasses over libiom_b200.so.
//
// Structure follows what the contract asks of a backend
// (docs/BACKEND_CONTRACT/implementing-a-backend.md:1-25) and the lifetime
// protocol the reference CPU queue demonstrates (src/cpu/queue.cpp:230-395):
// every hook hands its validated snapshot to the common submit_* helper; the
// dispatch callback launches the kernel on the queue's stream, records an
// event, and queues a retirement task; one worker thread per queue waits for
// the event, releases the registry entries and completes the sequence.
// Descriptors go to the kernels by value, so there is no metadata arena and no
// per-operation upload (the reference CUDA queue needs both,
// src/shared/gpu_queue_operations.inl:756-818).
#include "iom_b200_backend.hpp"

#include <cuda_runtime_api.h>

#include <array>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <mutex>
#include <new>
#include <span>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "iom/alloc.hpp"
#include "iom/detail/gpu_arena_config.hpp"
#include "iom/detail/outstanding_work_cleanup.hpp"
#include "iom/detail/outstanding_work_registry.hpp"
#include "iom/gpu_algorithm.hpp"
#include "iom_b200.h"
#include "iom_internal.hpp"   // reference src/: detail::UnsupportedOperation

namespace iom {
namespace {

constexpr DataType kLeaves[] = {
        DataType::BOOL, DataType::I2, DataType::U2, DataType::I4, DataType::U4,
        DataType::I8, DataType::U8, DataType::I16, DataType::U16, DataType::I32,
        DataType::U32, DataType::I64, DataType::U64, DataType::F4_E2M1,
        DataType::F6_E2M3, DataType::F6_E3M2, DataType::F8_E4M3FN, DataType::F8_E5M2,
        DataType::F8_E8M0, DataType::F16, DataType::BF16, DataType::F32, DataType::F64};

void check_cuda(const char* what, cudaError_t status) {
    if (status == cudaSuccess) return;
    if (status == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        throw std::bad_alloc();
    }
    const std::string text = std::string(what) + ": " + cudaGetErrorString(status);
    (void)cudaGetLastError();
    throw std::runtime_error(text);
}

// C-ABI status -> the exception category the facade maps to an oid
// (src/device_ops.cpp:422-439).
[[noreturn]] void throw_status(int status) {
    const std::string text = iomb_last_error();
    switch (status) {
        case IOMB_ERR_INVALID_ARGUMENT: throw std::invalid_argument(text);
        case IOMB_ERR_UNSUPPORTED: throw detail::UnsupportedOperation();
        case IOMB_ERR_OVERFLOW: throw std::overflow_error(text);
        case IOMB_ERR_RESOURCE_EXHAUSTED: throw std::bad_alloc();
        default: throw std::runtime_error(text);
    }
}

void check_status(int status) {
    if (status != IOMB_OK) throw_status(status);
}

template <typename Snapshot>
iomb_view to_view(const Snapshot& snapshot) {
    iomb_view view{};
    view.base = snapshot.native_handle;
    // The owner's extent, not the view's: a sliced view reaches beyond the
    // storage a dense tensor of its own shape would need.
    view.storage_bytes = snapshot.owner_identity->view().spec().tiled_storage_nbytes();
    view.dtype = static_cast<std::uint32_t>(snapshot.spec.data_type);
    const auto dims = snapshot.spec.shape.dimensions();
    view.rank = static_cast<std::uint32_t>(dims.size());
    for (std::size_t i = 0; i < dims.size(); ++i) view.dims[i] = dims[i];
    view.plane_offset = snapshot.plane_offset;
    for (std::size_t i = 0; i < snapshot.plane_strides.size() && i < IOMB_MAX_LEADING; ++i) {
        view.plane_strides[i] = snapshot.plane_strides[i];
    }
    return view;
}

iomb_view to_view(const TensorView& tensor_view) {
    iomb_view view{};
    view.base = const_cast<void*>(tensor_view.native_handle());
    view.storage_bytes = tensor_view.owner_identity()->view().spec().tiled_storage_nbytes();
    view.dtype = static_cast<std::uint32_t>(tensor_view.spec().data_type);
    const auto dims = tensor_view.spec().shape.dimensions();
    view.rank = static_cast<std::uint32_t>(dims.size());
    for (std::size_t i = 0; i < dims.size(); ++i) view.dims[i] = dims[i];
    view.plane_offset = tensor_view.plane_offset();
    const auto strides = tensor_view.plane_strides();
    for (std::size_t i = 0; i < strides.size() && i < IOMB_MAX_LEADING; ++i) {
        view.plane_strides[i] = strides[i];
    }
    return view;
}

// Fixed-capacity snapshot of cache_append (include/iom/iom.hpp:407-426).
template <typename Snapshot>
iomb_view to_view_fixed(const Snapshot& snapshot) {
    iomb_view view{};
    view.base = snapshot.native_handle;
    view.dtype = static_cast<std::uint32_t>(snapshot.data_type);
    view.rank = static_cast<std::uint32_t>(snapshot.rank);
    for (std::size_t i = 0; i < snapshot.rank; ++i) view.dims[i] = snapshot.dimensions[i];
    view.plane_offset = snapshot.plane_offset;
    for (std::size_t i = 0; i + 2 < snapshot.rank; ++i) {
        view.plane_strides[i] = snapshot.plane_strides[i];
    }
    view.storage_bytes = snapshot.owner_identity->view().spec().tiled_storage_nbytes();
    return view;
}

class B200Device;

class B200Workspace final : public RawWorkspace {
public:
    B200Workspace(B200Device& device, void* address, std::size_t bytes);
    ~B200Workspace() override;

private:
    [[nodiscard]] void* workspace_address() const noexcept override { return address_; }
    B200Device& device_;
    void* address_;
};

class B200Device final : public Device {
public:
    B200Device(std::uint32_t ordinal, DeviceMemoryConfig memory, QueueConfig queue_config)
            : Device(queue_config), ordinal_(ordinal), arena_bytes_(memory.tensor_arena_bytes) {
        (void)detail::valid_tensor_arena_bytes(memory.tensor_arena_bytes);
        int count = 0;
        check_cuda("cudaGetDeviceCount", cudaGetDeviceCount(&count));
        if (static_cast<int>(ordinal) >= count) {
            throw std::invalid_argument("B200 device ordinal does not exist");
        }
        activate();
        check_cuda("cudaMalloc(tensor arena)", cudaMalloc(&arena_, arena_bytes_));
        try {
            allocator_ = std::make_unique<ListAllocator>(arena_, arena_bytes_, 256);
            check_cuda("cudaStreamCreate(transfer)",
                       cudaStreamCreateWithFlags(&transfer_stream_, cudaStreamNonBlocking));
        } catch (...) {
            (void)cudaFree(arena_);
            throw;
        }
    }

    ~B200Device() override {
        if (transfer_stream_ != nullptr) (void)cudaStreamDestroy(transfer_stream_);
        for (const RopeTable& table : rope_tables_) (void)cudaFree(table.device);
        allocator_.reset();
        if (arena_ != nullptr) (void)cudaFree(arena_);
    }

    void activate() const { check_cuda("cudaSetDevice", cudaSetDevice(static_cast<int>(ordinal_))); }

    [[nodiscard]] BackendKind backend_kind() const noexcept override { return BackendKind::CUDA; }
    [[nodiscard]] std::uint32_t backend_device() const noexcept override { return ordinal_; }
    [[nodiscard]] std::span<const DataType> supported_data_types() const noexcept override {
        return kLeaves;
    }
    [[nodiscard]] detail::RegistryState& registry_state() noexcept { return registry_state_; }

    [[nodiscard]] void* allocate(std::size_t bytes) {
        std::lock_guard<std::mutex> lock(allocator_mutex_);
        void* address = allocator_->alloc(bytes);
        if (address == nullptr) throw std::bad_alloc();
        return address;
    }
    void release(void* address) noexcept {
        std::lock_guard<std::mutex> lock(allocator_mutex_);
        try {
            allocator_->free(address);
        } catch (...) {
        }
    }
    [[nodiscard]] Allocator& data_allocator() noexcept { return *allocator_; }
    [[nodiscard]] cudaStream_t transfer_stream() const noexcept { return transfer_stream_; }
    [[nodiscard]] std::mutex& transfer_mutex() noexcept { return transfer_mutex_; }

    // Rotary cache: device table of (cos, sin) for positions 0 .. rows-1 of one
    // (theta, width), built on the host by iomb_rope_angles and grown by doubling.
    // Tables live outside the tensor arena and until the device goes away, because
    // queued work may still read a table that a longer one has replaced.
    [[nodiscard]] const float* rope_table(double theta, std::size_t width, std::size_t positions) {
        std::lock_guard<std::mutex> lock(rope_mutex_);
        const float narrowed = static_cast<float>(theta);
        std::uint32_t theta_bits = 0;
        std::memcpy(&theta_bits, &narrowed, sizeof theta_bits);
        for (const RopeTable& table : rope_tables_) {
            if (table.theta_bits == theta_bits && table.width == width && table.rows >= positions) {
                return table.device;
            }
        }
        std::size_t rows = 256;
        while (rows < positions) rows *= 2;
        const std::size_t count = rows * (width / 2) * 2;
        std::vector<float> host(count);
        check_status(iomb_rope_angles(host.data(), 0, rows, width, theta));
        activate();
        void* allocation = nullptr;
        check_cuda("cudaMalloc(rope table)", cudaMalloc(&allocation, count * sizeof(float)));
        float* device = static_cast<float*>(allocation);
        const cudaError_t copied = cudaMemcpy(device, host.data(), count * sizeof(float),
                                              cudaMemcpyHostToDevice);
        if (copied != cudaSuccess) {
            (void)cudaFree(device);
            check_cuda("cudaMemcpy(rope table)", copied);
        }
        rope_tables_.push_back(RopeTable{theta_bits, width, rows, device});
        return device;
    }

    [[nodiscard]] std::unique_ptr<Tensor> create_tensor(const TensorSpec& spec) override;
    [[nodiscard]] std::unique_ptr<RawWorkspace> create_workspace(std::size_t bytes) override {
        if (bytes == 0) return std::make_unique<B200Workspace>(*this, nullptr, 0);
        void* address = allocate(bytes);
        try {
            return std::make_unique<B200Workspace>(*this, address, bytes);
        } catch (...) {
            release(address);
            throw;
        }
    }
    [[nodiscard]] std::unique_ptr<DeviceOps> create_ops() override;

private:
    std::uint32_t ordinal_;
    std::size_t arena_bytes_;
    void* arena_ = nullptr;
    std::unique_ptr<ListAllocator> allocator_;
    std::mutex allocator_mutex_;
    cudaStream_t transfer_stream_ = nullptr;
    std::mutex transfer_mutex_;
    detail::RegistryState registry_state_;
    struct RopeTable {
        std::uint32_t theta_bits;
        std::size_t width;
        std::size_t rows;
        float* device;
    };
    std::vector<RopeTable> rope_tables_;
    std::mutex rope_mutex_;
};

B200Workspace::B200Workspace(B200Device& device, void* address, std::size_t bytes)
        : RawWorkspace(device, bytes), device_(device), address_(address) {}

B200Workspace::~B200Workspace() {
    if (address_ != nullptr) device_.release(address_);
}

// Checks the {staging, 32} host-transfer workspace the contract makes mandatory
// (test/backend/backend_conformance_memory.hpp:72-135) and returns its address.
void* staging_address(const B200Device& device, const RawWorkspaceView& workspace,
                      std::size_t logical_bytes) {
    const std::size_t needed = gpu_algorithm::compute_staging_size(logical_bytes);
    if (needed == 0) return nullptr;
    if (workspace.empty() || &workspace.device() != &device
            || !device.owns_workspace(workspace.owner_identity())) {
        throw std::invalid_argument("host transfer requires a live staging workspace of this device");
    }
    if (workspace.byte_size() < needed) {
        throw std::invalid_argument("host transfer staging workspace is too small");
    }
    void* address = detail::WorkspaceValidation::address(workspace);
    if (reinterpret_cast<std::uintptr_t>(address) % 32 != 0) {
        throw std::invalid_argument("host transfer staging workspace is misaligned");
    }
    return address;
}

class B200Tensor final : public Tensor {
public:
    B200Tensor(const TensorSpec& spec, B200Device& device) : Tensor(spec, device), device_(device) {
        const std::size_t bytes = view().spec().tiled_storage_nbytes();
        address_ = device_.allocate(bytes);
        try {
            device_.activate();
            check_cuda("cudaMemset", cudaMemset(address_, 0, bytes));
            check_cuda("cudaDeviceSynchronize", cudaDeviceSynchronize());
        } catch (...) {
            device_.release(address_);
            address_ = nullptr;
            throw;
        }
    }

    ~B200Tensor() noexcept override {
        if (address_ == nullptr) return;
        const std::size_t bytes = view().spec().tiled_storage_nbytes();
        detail::RegistryState& state = device_.registry_state();
        // Storage with unproven outstanding work is parked, never recycled
        // (the rule of src/cuda/device_tensor.cpp:105-131).
        detail::release_or_quarantine(
                state.registry, address_,
                [this, bytes, &state]() noexcept {
                    try {
                        state.quarantine.emplace<detail::AllocatorCleanupAction>(
                                device_.data_allocator(), address_, bytes);
                    } catch (...) {
                    }
                    address_ = nullptr;
                },
                [this]() noexcept {
                    device_.release(address_);
                    address_ = nullptr;
                });
    }

private:
    [[nodiscard]] void* storage_handle() noexcept override { return address_; }
    [[nodiscard]] WorkspaceRequirements host_transfer_workspace_requirements(
            std::size_t logical_bytes) const override {
        return {gpu_algorithm::compute_staging_size(logical_bytes), 32};
    }

    void region_from_host(const TensorView& destination, std::span<const std::byte> source,
                          RawWorkspaceView workspace) override {
        std::lock_guard<std::mutex> lock(device_.transfer_mutex());
        device_.activate();
        void* staging = staging_address(device_, workspace, source.size());
        const cudaStream_t stream = device_.transfer_stream();
        check_cuda("cudaMemcpyAsync(H2D)",
                   cudaMemcpyAsync(staging, source.data(), source.size(),
                                   cudaMemcpyHostToDevice, stream));
        const iomb_view view = to_view(destination);
        check_status(iomb_scatter(&view, staging, stream));
        check_cuda("cudaStreamSynchronize", cudaStreamSynchronize(stream));
    }

    void region_to_host(const TensorView& source, std::span<std::byte> destination,
                        RawWorkspaceView workspace) const override {
        std::lock_guard<std::mutex> lock(device_.transfer_mutex());
        device_.activate();
        void* staging = staging_address(device_, workspace, destination.size());
        const cudaStream_t stream = device_.transfer_stream();
        const iomb_view view = to_view(source);
        check_status(iomb_gather(&view, staging, stream));
        check_cuda("cudaMemcpyAsync(D2H)",
                   cudaMemcpyAsync(destination.data(), staging, destination.size(),
                                   cudaMemcpyDeviceToHost, stream));
        check_cuda("cudaStreamSynchronize", cudaStreamSynchronize(stream));
    }

    B200Device& device_;
    void* address_ = nullptr;
};

std::unique_ptr<Tensor> B200Device::create_tensor(const TensorSpec& spec) {
    return std::make_unique<B200Tensor>(spec, *this);
}

// ---- operation queue ----------------------------------------------------------

class B200Queue final : public DeviceOps {
    struct Retirement {
        std::function<void()> work;
    };

public:
    explicit B200Queue(B200Device& device)
            : DeviceOps(device), device_(&device),
              registry_queue_id_(detail::allocate_queue_id(device.registry_state())) {
        device_->activate();
        check_cuda("cudaStreamCreate", cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
        // One event per in-flight credit (+1 so a ring slot is never reused
        // while its retirement is still running); one pinned status cell each.
        const std::size_t credits = device.queue_config().max_in_flight_per_queue + 1;
        try {
            events_.resize(credits, nullptr);
            for (cudaEvent_t& event : events_) {
                check_cuda("cudaEventCreate",
                           cudaEventCreateWithFlags(&event, cudaEventDisableTiming));
            }
            check_cuda("cudaMallocHost",
                       cudaMallocHost(reinterpret_cast<void**>(&status_cells_),
                                      credits * sizeof(std::uint32_t)));
        } catch (...) {
            destroy_native();
            throw;
        }
        worker_ = std::thread([this] { run_worker(); });
    }

    ~B200Queue() override {
        close_and_drain();
        {
            std::lock_guard<std::mutex> lock(worker_mutex_);
            worker_shutdown_ = true;
        }
        worker_cv_.notify_all();
        if (worker_.joinable()) worker_.join();
        device_->registry_state().registry.invalidate_entries_for_queue(registry_queue_id_);
        destroy_native();
    }

    [[nodiscard]] cudaStream_t stream() const noexcept { return stream_; }

    // Extension entry (see iom_b200_backend.hpp).
    oid add_rmsnorm(const TensorView& x, const TensorView& residual, const TensorView& scale,
                    TensorView& sum, TensorView& out, float eps) {
        try {
            validate_views(queue_device(), {&x, &residual, &scale, &sum, &out});
            const iomb_view vx = to_view(x), vr = to_view(residual), vw = to_view(scale),
                            vs = to_view(sum), vo = to_view(out);
            std::lock_guard<std::mutex> order(submission_order_mutex_);
            return submit([this, vx, vr, vw, vs, vo, eps](std::uint64_t sequence) {
                device_->activate();
                check_status(iomb_add_rmsnorm(&vx, &vr, &vw, &vs, &vo, eps, IOMB_RMS_LANES16, stream_));
                retire(sequence, [] {}, nullptr);
            });
        } catch (const std::invalid_argument&) {
            return to_oid(OidError::InvalidArgument);
        } catch (const detail::UnsupportedOperation&) {
            return to_oid(OidError::Unsupported);
        } catch (const std::bad_alloc&) {
            return to_oid(OidError::ResourceExhausted);
        } catch (...) {
            return to_oid(OidError::DeviceError);
        }
    }

    // Extension entry (see iom_b200_backend.hpp). `activated` may be null.
    oid silu_mul(const TensorView& x, const TensorView& up, TensorView* activated, TensorView& out) {
        try {
            if (activated != nullptr) {
                validate_views(queue_device(), {&x, &up, activated, &out});
            } else {
                validate_views(queue_device(), {&x, &up, &out});
            }
            const iomb_view vx = to_view(x), vu = to_view(up), vo = to_view(out);
            const bool stores_activated = activated != nullptr;
            const iomb_view va = stores_activated ? to_view(*activated) : iomb_view{};
            std::lock_guard<std::mutex> order(submission_order_mutex_);
            return submit([this, vx, vu, va, vo, stores_activated](std::uint64_t sequence) {
                device_->activate();
                check_status(iomb_silu_mul(&vx, &vu, stores_activated ? &va : nullptr, &vo, stream_));
                retire(sequence, [] {}, nullptr);
            });
        } catch (const std::invalid_argument&) {
            return to_oid(OidError::InvalidArgument);
        } catch (const detail::UnsupportedOperation&) {
            return to_oid(OidError::Unsupported);
        } catch (const std::bad_alloc&) {
            return to_oid(OidError::ResourceExhausted);
        } catch (...) {
            return to_oid(OidError::DeviceError);
        }
    }

    // Extension entries (see iom_b200_backend.hpp): one admission / submission /
    // failure-mapping path for calls that take raw device addresses besides views.
    template <typename Launch>
    oid extension(std::initializer_list<const TensorView*> views, Launch launch) {
        try {
            validate_views(queue_device(), views);
            std::lock_guard<std::mutex> order(submission_order_mutex_);
            return submit([this, launch](std::uint64_t sequence) {
                device_->activate();
                check_status(launch(stream_));
                retire(sequence, [] {}, nullptr);
            });
        } catch (const std::invalid_argument&) {
            return to_oid(OidError::InvalidArgument);
        } catch (const detail::UnsupportedOperation&) {
            return to_oid(OidError::Unsupported);
        } catch (const std::bad_alloc&) {
            return to_oid(OidError::ResourceExhausted);
        } catch (...) {
            return to_oid(OidError::DeviceError);
        }
    }

    oid cast(const TensorView& source, TensorView& destination) {
        const iomb_view vs = to_view(source), vd = to_view(destination);
        return extension({&source, &destination},
                         [vs, vd](cudaStream_t stream) { return iomb_cast(&vs, &vd, stream); });
    }

    oid cache_append_batched(const TensorView& source, TensorView& destination,
                             const std::uint32_t* positions, std::uint32_t* status) {
        const iomb_view vs = to_view(source), vd = to_view(destination);
        return extension({&source, &destination}, [vs, vd, positions, status](cudaStream_t stream) {
            return iomb_cache_append_batched(&vs, &vd, positions, status, stream);
        });
    }

    oid sumsq(const TensorView& x, void* scratch, float* result) {
        const iomb_view vx = to_view(x);
        return extension({&x}, [vx, scratch, result](cudaStream_t stream) {
            return iomb_sumsq(&vx, scratch, result, stream);
        });
    }

    // stage: 0 scale/mask, 1 softmax, 2 both (scores only read), 3 both (scaled scores stored)
    oid sdpa_stage(int stage, const b200::SdpaStages& s) {
        const iomb_sdpa_stages request{s.scores, s.probability, s.planes, s.Hq, s.Hkv,
                                       s.R, s.C, s.D, s.a, s.L};
        return extension({}, [stage, request](cudaStream_t stream) {
            switch (stage) {
                case 0: return iomb_sdpa_scale_mask(&request, stream);
                case 1: return iomb_sdpa_softmax(&request, stream);
                default: return iomb_sdpa_scale_mask_softmax(&request, stage == 3 ? 1 : 0, stream);
            }
        });
    }

    oid sdpa_canonicalize_output(TensorView& out) {
        const iomb_view vo = to_view(out);
        return extension({&out}, [vo](cudaStream_t stream) {
            return iomb_sdpa_canonicalize_output(&vo, stream);
        });
    }

protected:
    [[nodiscard]] std::string_view backend_label() const noexcept override { return "B200"; }

    oid copy_impl(const TensorView& source, TensorView& destination) override {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        return submit_copy(
                source, destination, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const CopyRequest& request,
                       detail::EntryRegistration entries) {
                    auto release = [this, entries](bool failed) {
                        const detail::SequenceOutcome outcome{entries.source, entries.destination,
                                                              nullptr, true};
                        (void)detail::release_or_invalidate_entries(
                                device_->registry_state().registry, outcome, failed, !failed);
                    };
                    try {
                        if (!request.no_op) {
                            device_->activate();
                            const iomb_view src = to_view(request.source);
                            const iomb_view dst = to_view(request.destination);
                            check_status(iomb_copy(&src, &dst, stream_));
                        }
                        retire(sequence, [release] { release(false); }, nullptr);
                    } catch (...) {
                        release(true);
                        throw;
                    }
                });
    }

    static_assert(static_cast<int>(BinaryOperation::Add) == IOMB_ADD
                          && static_cast<int>(BinaryOperation::Mul) == IOMB_MUL
                          && static_cast<int>(BinaryOperation::Sub) == IOMB_SUB
                          && static_cast<int>(BinaryOperation::Div) == IOMB_DIV,
                  "BinaryOperation and iomb_binary_op must share their ordinals");

    oid binary_impl(const BinaryRequest& request) override {
        switch (request.out.spec.data_type) {
            case DataType::I8: case DataType::U8: case DataType::I16: case DataType::U16:
            case DataType::I32: case DataType::U32: case DataType::I64: case DataType::U64:
            case DataType::I2: case DataType::U2: case DataType::I4: case DataType::U4:
            case DataType::F4_E2M1: case DataType::F6_E2M3: case DataType::F6_E3M2:
            case DataType::F8_E4M3FN: case DataType::F8_E5M2:
            case DataType::F16: case DataType::BF16: case DataType::F32: break;
            default: throw detail::UnsupportedOperation();
        }
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        return submit_binary(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const BinaryRequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    launch_three_owner(sequence, entries, captured.workspace_lease, [&] {
                        const iomb_view lhs = to_view(captured.lhs), rhs = to_view(captured.rhs),
                                        out = to_view(captured.out);
                        // BinaryOperation and iomb_binary_op share their ordinals.
                        check_status(iomb_binary(static_cast<int>(captured.operation), &lhs, &rhs,
                                                 &out, stream_));
                    });
                });
    }

    [[nodiscard]] bool rmsnorm_supported(DataType data_type) const override {
        return data_type == DataType::BF16 || data_type == DataType::F32;
    }

    oid rmsnorm_impl(const RmsnormRequest& request) override {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        return submit_rmsnorm(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const RmsnormRequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    launch_three_owner(sequence, entries, {}, [&] {
                        const iomb_view x = to_view(captured.x), w = to_view(captured.scale),
                                        out = to_view(captured.out);
                        check_status(iomb_rmsnorm(&x, &w, &out, captured.epsilon,
                                                  IOMB_RMS_LANES16, stream_));
                    });
                });
    }

    [[nodiscard]] WorkspaceRequirements embedding_workspace_requirements_impl(
            const TensorView& table, const TensorView& indices, const TensorView&) override {
        if (detail::leaf_bits(indices.spec().data_type) % 8 != 0) {
            throw detail::UnsupportedOperation();
        }
        // First u32 of the range is the status word (0 ok / 1 invalid id),
        // docs/BACKEND_CONTRACT/embedding-lookup.md:178-209.
        return {32, 32};
    }

    oid embedding_impl(const EmbeddingRequest& request) override {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        return submit_embedding(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const EmbeddingRequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    auto* status = static_cast<std::uint32_t*>(
                            detail::WorkspaceValidation::address(captured.workspace));
                    std::uint32_t* cell = status_cells_ + sequence % events_.size();
                    launch_three_owner(
                            sequence, entries, captured.workspace_lease,
                            [&] {
                                const iomb_view table = to_view(captured.table),
                                                ids = to_view(captured.indices),
                                                out = to_view(captured.out);
                                check_status(iomb_embedding(&table, &ids, &out, status, stream_));
                                *cell = 0;
                                check_cuda("cudaMemcpyAsync(status)",
                                           cudaMemcpyAsync(cell, status, sizeof(std::uint32_t),
                                                           cudaMemcpyDeviceToHost, stream_));
                            },
                            cell);
                });
    }

    [[nodiscard]] WorkspaceRequirements cache_append_workspace_requirements(
            const CacheAppendRequest& request) override {
        (void)request;   // every leaf width (8..64 bits, and 2, 4, 6 bits) has a kernel
        return {0, 1};
    }

    oid cache_append_impl(const CacheAppendRequest& request) override {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        return submit_cache_append(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const CacheAppendRequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    launch_three_owner(sequence, entries, captured.workspace_lease, [&] {
                        const iomb_view src = to_view_fixed(captured.source),
                                        dst = to_view_fixed(captured.destination);
                        check_status(iomb_cache_append(&src, &dst, captured.a, stream_));
                    });
                });
    }

    [[nodiscard]] WorkspaceRequirements silu_workspace_requirements_impl(
            const SiLURequest& request) override {
        if (request.x.data_type != DataType::BF16 && request.x.data_type != DataType::F32) {
            throw detail::UnsupportedOperation();
        }
        return {0, 1};
    }

    oid silu_impl(const SiLURequest& request) override {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        return submit_silu(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const SiLURequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    launch_three_owner(sequence, entries, {}, [&] {
                        const iomb_view x = to_view_fixed(captured.x), y = to_view_fixed(captured.y);
                        check_status(iomb_silu(&x, &y, stream_));
                    });
                });
    }

    [[nodiscard]] WorkspaceRequirements rope_workspace_requirements(
            const RopeRequest& request) override {
        if (request.x.data_type != DataType::BF16 && request.x.data_type != DataType::F32) {
            throw detail::UnsupportedOperation();
        }
        return {0, 1};
    }

    oid rope_impl(const RopeRequest& request) override {
        // The table covers positions 0 .. a + R - 1; row a is where this request starts.
        const std::size_t rows = request.x.dimensions[request.x.rank - 2];
        const std::size_t width = request.x.dimensions[request.x.rank - 1];
        const float* table = device_->rope_table(request.theta, width, request.a + rows);
        const float* first = table + request.a * (width / 2) * 2;
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        return submit_rope(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this, first](std::uint64_t sequence, const RopeRequest& captured,
                              detail::BinaryEntryRegistration entries) {
                    launch_three_owner(sequence, entries, {}, [&] {
                        const iomb_view x = to_view_fixed(captured.x), out = to_view_fixed(captured.out);
                        check_status(iomb_rope(&x, &out, captured.a, first, stream_));
                    });
                });
    }

private:
    // Completion proof handed to the owner registry: draining this queue's
    // stream proves every registered operation has finished.
    static detail::FenceResult fence_drain(const detail::Fence& fence) noexcept {
        cudaStream_t stream = nullptr;
        std::memcpy(&stream, fence.storage, sizeof stream);
        return cudaStreamSynchronize(stream) == cudaSuccess
                ? detail::FenceResult::success()
                : detail::FenceResult::failed(std::make_exception_ptr(
                          std::runtime_error("B200 queue stream failed to drain")));
    }

    [[nodiscard]] detail::Fence fence() const noexcept {
        detail::Fence result;
        std::memcpy(result.storage, &stream_, sizeof stream_);
        result.invoke = &fence_drain;
        return result;
    }

    // Launches through `launch`, then schedules retirement; on a launch
    // failure the registrations are dropped and the exception reaches the
    // facade (synchronous error) or the retained-failure path.
    template <typename Launch>
    void launch_three_owner(std::uint64_t sequence, detail::BinaryEntryRegistration entries,
                            detail::WorkspaceLease lease, Launch&& launch,
                            const std::uint32_t* status_cell = nullptr) {
        auto release = [this, entries, lease](bool failed) {
            (void)detail::release_or_invalidate_binary_entries(
                    device_->registry_state().registry, entries, failed, !failed);
            detail::complete_workspace_lease(device_->registry_state(), lease, true);
        };
        try {
            device_->activate();
            launch();
            retire(sequence, [release] { release(false); }, status_cell);
        } catch (...) {
            device_->registry_state().registry.remove_entries(
                    std::span<const detail::EntryId>(entries.entries.data(), entries.count));
            detail::complete_workspace_lease(device_->registry_state(), lease, true);
            throw;
        }
    }

    // Records the completion event and hands the sequence to the worker.
    void retire(std::uint64_t sequence, std::function<void()> release,
                const std::uint32_t* status_cell) {
        cudaEvent_t event = events_[sequence % events_.size()];
        check_cuda("cudaEventRecord", cudaEventRecord(event, stream_));
        {
            std::lock_guard<std::mutex> lock(worker_mutex_);
            if (worker_shutdown_) throw std::logic_error("B200 queue worker is shut down");
            worker_tasks_.push_back(Retirement{[this, sequence, event, status_cell,
                                                release = std::move(release)] {
                std::exception_ptr failure;
                const cudaError_t status = cudaEventSynchronize(event);
                if (status != cudaSuccess) {
                    failure = std::make_exception_ptr(std::runtime_error(
                            std::string("B200 operation failed: ") + cudaGetErrorString(status)));
                } else if (status_cell != nullptr && *status_cell != 0) {
                    // An invalid id is a retained invalid_argument
                    // (src/shared/gpu_queue_operations.inl:1080-1095).
                    failure = std::make_exception_ptr(
                            std::invalid_argument("embedding index is negative or out of range"));
                }
                release();
                complete(sequence, std::move(failure));
            }});
        }
        worker_cv_.notify_one();
    }

    void run_worker() noexcept {
        (void)cudaSetDevice(static_cast<int>(device_->backend_device()));
        for (;;) {
            Retirement task;
            {
                std::unique_lock<std::mutex> lock(worker_mutex_);
                worker_cv_.wait(lock, [this] { return worker_shutdown_ || !worker_tasks_.empty(); });
                if (worker_tasks_.empty()) return;
                task = std::move(worker_tasks_.front());
                worker_tasks_.pop_front();
            }
            try {
                task.work();
            } catch (...) {
            }
        }
    }

    void destroy_native() noexcept {
        for (cudaEvent_t event : events_) {
            if (event != nullptr) (void)cudaEventDestroy(event);
        }
        events_.clear();
        if (status_cells_ != nullptr) (void)cudaFreeHost(status_cells_);
        status_cells_ = nullptr;
        if (stream_ != nullptr) (void)cudaStreamDestroy(stream_);
        stream_ = nullptr;
    }

    B200Device* device_;
    detail::QueueId registry_queue_id_;
    cudaStream_t stream_ = nullptr;
    std::vector<cudaEvent_t> events_;
    std::uint32_t* status_cells_ = nullptr;
    std::mutex submission_order_mutex_;
    std::mutex worker_mutex_;
    std::condition_variable worker_cv_;
    std::deque<Retirement> worker_tasks_;
    bool worker_shutdown_ = false;
    std::thread worker_;
};

std::unique_ptr<DeviceOps> B200Device::create_ops() {
    return std::make_unique<B200Queue>(*this);
}

}  // namespace

std::unique_ptr<Device> make_b200_device(
        std::uint32_t ordinal, DeviceMemoryConfig memory_config, QueueConfig queue_config) {
    return std::make_unique<B200Device>(ordinal, memory_config, queue_config);
}

namespace b200 {

oid add_rmsnorm(DeviceOps& queue, const TensorView& x, const TensorView& residual,
                const TensorView& scale, TensorView& sum, TensorView& out, float eps) {
    auto* native = dynamic_cast<B200Queue*>(&queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->add_rmsnorm(x, residual, scale, sum, out, eps);
}

oid cast(DeviceOps& queue, const TensorView& source, TensorView& destination) {
    auto* native = dynamic_cast<B200Queue*>(&queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->cast(source, destination);
}

oid cache_append_batched(DeviceOps& queue, const TensorView& source, TensorView& destination,
                         const std::uint32_t* positions, std::uint32_t* status) {
    auto* native = dynamic_cast<B200Queue*>(&queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->cache_append_batched(source, destination, positions, status);
}

oid sumsq(DeviceOps& queue, const TensorView& x, void* scratch, float* result) {
    auto* native = dynamic_cast<B200Queue*>(&queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->sumsq(x, scratch, result);
}

namespace {
oid sdpa_stage_of(DeviceOps& queue, int stage, const SdpaStages& stages) {
    auto* native = dynamic_cast<B200Queue*>(&queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->sdpa_stage(stage, stages);
}
}  // namespace

oid sdpa_scale_mask(DeviceOps& queue, const SdpaStages& stages) { return sdpa_stage_of(queue, 0, stages); }
oid sdpa_softmax(DeviceOps& queue, const SdpaStages& stages) { return sdpa_stage_of(queue, 1, stages); }
oid sdpa_scale_mask_softmax(DeviceOps& queue, const SdpaStages& stages, bool keep_scores) {
    return sdpa_stage_of(queue, keep_scores ? 3 : 2, stages);
}
oid sdpa_canonicalize_output(DeviceOps& queue, TensorView& out) {
    auto* native = dynamic_cast<B200Queue*>(&queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->sdpa_canonicalize_output(out);
}

std::size_t sumsq_scratch_bytes() { return static_cast<std::size_t>(iomb_sumsq_scratch_bytes()); }

oid silu_mul(DeviceOps& queue, const TensorView& x, const TensorView& up, TensorView* activated,
             TensorView& out) {
    auto* native = dynamic_cast<B200Queue*>(&queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->silu_mul(x, up, activated, out);
}

}  // namespace b200
}  // namespace iom
