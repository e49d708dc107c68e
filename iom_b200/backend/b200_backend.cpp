// B200 backend for IOM's backend contract: Device / Tensor / RawWorkspace /
// DeviceOps subclasses over libiom_b200.so.
//
// Structure follows what the contract asks of a backend
// (docs/BACKEND_CONTRACT/implementing-a-backend.md:1-25) and the lifetime
// protocol of the reference's GPU queue (src/shared/gpu_queue_operations.inl):
// every hook hands its validated snapshot to the common submit_* helper; the
// dispatch callback launches the kernel on the queue's stream, records an
// event taken from a fixed set sized by the credit count, and publishes a
// plain-data retirement record into a fixed ring; one worker thread per queue
// waits for the event, releases the registry entries and completes the
// sequence. Nothing is allocated per operation on this side of the facade.
// Descriptors go to the kernels by value, so there is no metadata arena and no
// per-operation upload (the reference CUDA queue needs both,
// src/shared/gpu_queue_operations.inl:756-818).
//
// Completion proof (src/shared/gpu_queue_operations.inl:1030-1051): the recorded
// event; if it cannot be recorded, a drain of the stream; if that fails too the
// completion is unknown: the operation fails, its owner entries are invalidated,
// its workspace lease and its event are quarantined (never reused).
#include "iom_b200_backend.hpp"

#include <cuda_runtime_api.h>

#include <array>
#include <atomic>
#include <cstring>
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

// Accumulation order behind the facade. BF16 takes the lane order: bit-identical to the
// reference's AVX-512 BF16 build (src/cpu/avx512_bf16_rmsnorm_reduction.cpp:69-81) and at
// most one code from the portable one. F32 has one order in the reference, sequential
// (src/cpu/queue.cpp:1187-1196), and takes it: bit-identical.
int facade_order(DataType data_type) {
    return data_type == DataType::F32 ? IOMB_RMS_SEQUENTIAL : IOMB_RMS_LANES16;
}

// ---- host-side failure injection (src/cuda/copy.cu:54-88,728-737) ---------------------

std::atomic<b200::SubmissionFault> g_fault{b200::SubmissionFault::none};
std::atomic<int> g_event_record_failures{0};
std::atomic<int> g_stream_sync_failures{0};

bool consume_fault(b200::SubmissionFault point) noexcept {
    if (point == b200::SubmissionFault::event_record
            || point == b200::SubmissionFault::stream_synchronize) {
        auto& failures = point == b200::SubmissionFault::event_record
                ? g_event_record_failures : g_stream_sync_failures;
        int remaining = failures.load(std::memory_order_acquire);
        while (remaining > 0
               && !failures.compare_exchange_weak(remaining, remaining - 1,
                                                  std::memory_order_acq_rel)) {
        }
        return remaining > 0;
    }
    b200::SubmissionFault expected = point;
    return g_fault.compare_exchange_strong(expected, b200::SubmissionFault::none,
                                           std::memory_order_acq_rel);
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
    B200Device(std::uint32_t ordinal, DeviceMemoryConfig memory, QueueConfig queue_config,
               b200::Options options)
            : Device(queue_config), ordinal_(ordinal), arena_bytes_(memory.tensor_arena_bytes),
              rotary_bytes_(options.rotary_table_bytes / 32 * 32) {
        (void)detail::valid_tensor_arena_bytes(memory.tensor_arena_bytes);
        int count = 0;
        check_cuda("cudaGetDeviceCount", cudaGetDeviceCount(&count));
        if (static_cast<int>(ordinal) >= count) {
            throw std::invalid_argument("B200 device ordinal does not exist");
        }
        activate();
        // The only native allocations of this device's lifetime.
        check_cuda("cudaMalloc(tensor arena)", cudaMalloc(&arena_, arena_bytes_));
        try {
            if (rotary_bytes_ != 0) {
                check_cuda("cudaMalloc(rotary tables)", cudaMalloc(&rotary_, rotary_bytes_));
            }
            allocator_ = std::make_unique<ListAllocator>(arena_, arena_bytes_, 256);
            check_cuda("cudaStreamCreate(transfer)",
                       cudaStreamCreateWithFlags(&transfer_stream_, cudaStreamNonBlocking));
            check_cuda("cudaStreamCreate(download)",
                       cudaStreamCreateWithFlags(&download_stream_, cudaStreamNonBlocking));
            // One-time set-up of the kernel library on this device (function attributes,
            // the BF16 SiLU table), so that no operation does it later.
            check_status(iomb_prepare_device(transfer_stream_));
            check_cuda("cudaStreamSynchronize(set-up)", cudaStreamSynchronize(transfer_stream_));
        } catch (...) {
            if (transfer_stream_ != nullptr) (void)cudaStreamDestroy(transfer_stream_);
            if (download_stream_ != nullptr) (void)cudaStreamDestroy(download_stream_);
            if (rotary_ != nullptr) (void)cudaFree(rotary_);
            (void)cudaFree(arena_);
            throw;
        }
    }

    ~B200Device() override {
        if (transfer_stream_ != nullptr) (void)cudaStreamDestroy(transfer_stream_);
        if (download_stream_ != nullptr) (void)cudaStreamDestroy(download_stream_);
        // Parked storage goes back to the allocator while the allocator still exists
        // (src/cuda/device.cpp:106-116).
        registry_state_.quarantine.drain();
        allocator_.reset();
        if (rotary_ != nullptr) (void)cudaFree(rotary_);
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
    // Device-to-host transfers have a stream and a lock of their own, so that a thread
    // reading results back and a thread uploading the next inputs use both directions of
    // the link at once (each call is still synchronous for its caller).
    [[nodiscard]] cudaStream_t download_stream() const noexcept { return download_stream_; }
    [[nodiscard]] std::mutex& download_mutex() noexcept { return download_mutex_; }
    [[nodiscard]] std::mutex& transfer_mutex() noexcept { return transfer_mutex_; }

    // Rotary cache: device table of (cos, sin) for positions 0 .. rows-1 of one
    // (theta, width), computed on the host by iomb_rope_angles and placed in the region
    // reserved at construction. Tables are never moved or freed (queued work may still
    // read a table that a longer one has replaced); when the region is full the request
    // is refused with std::bad_alloc, as any exhausted fixed resource is.
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
        const std::size_t bytes = (count * sizeof(float) + 31) / 32 * 32;
        if (bytes > rotary_bytes_ - rotary_used_) throw std::bad_alloc();
        std::vector<float> host(count);
        check_status(iomb_rope_angles(host.data(), 0, rows, width, theta));
        float* device = reinterpret_cast<float*>(static_cast<unsigned char*>(rotary_) + rotary_used_);
        {
            std::lock_guard<std::mutex> transfer(transfer_mutex_);
            activate();
            check_cuda("cudaMemcpyAsync(rope table)",
                       cudaMemcpyAsync(device, host.data(), count * sizeof(float),
                                       cudaMemcpyHostToDevice, transfer_stream_));
            check_cuda("cudaStreamSynchronize(rope table)", cudaStreamSynchronize(transfer_stream_));
        }
        rotary_used_ += bytes;
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
    std::size_t rotary_bytes_;
    std::size_t rotary_used_ = 0;
    void* arena_ = nullptr;
    void* rotary_ = nullptr;
    std::unique_ptr<ListAllocator> allocator_;
    std::mutex allocator_mutex_;
    cudaStream_t transfer_stream_ = nullptr;
    cudaStream_t download_stream_ = nullptr;
    std::mutex download_mutex_;
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
    if (address_ == nullptr) return;
    // A range that unproven work may still use is parked like tensor storage.
    detail::RegistryState& state = device_.registry_state();
    const std::size_t bytes = byte_size();
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

// Drains the transfer stream; the stream_synchronize fault point substitutes a failure
// after the real drain, so nothing is left in flight.
void drain_transfer_stream(cudaStream_t stream) {
    const cudaError_t status = cudaStreamSynchronize(stream);
    if (consume_fault(b200::SubmissionFault::stream_synchronize)) {
        throw std::runtime_error("cudaStreamSynchronize: injected failure");
    }
    check_cuda("cudaStreamSynchronize", status);
}

class B200Tensor final : public Tensor {
public:
    B200Tensor(const TensorSpec& spec, B200Device& device) : Tensor(spec, device), device_(device) {
        const std::size_t bytes = view().spec().tiled_storage_nbytes();
        address_ = device_.allocate(bytes);
        try {
            // Zero-filled like the reference's tensors (src/cuda/device_tensor.cpp:81-103),
            // on the transfer stream: the other queues keep running.
            std::lock_guard<std::mutex> lock(device_.transfer_mutex());
            device_.activate();
            const cudaStream_t stream = device_.transfer_stream();
            check_cuda("cudaMemsetAsync", cudaMemsetAsync(address_, 0, bytes, stream));
            check_cuda("cudaStreamSynchronize", cudaStreamSynchronize(stream));
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
        drain_transfer_stream(stream);
    }

    void region_to_host(const TensorView& source, std::span<std::byte> destination,
                        RawWorkspaceView workspace) const override {
        std::lock_guard<std::mutex> lock(device_.download_mutex());
        device_.activate();
        void* staging = staging_address(device_, workspace, destination.size());
        const cudaStream_t stream = device_.download_stream();
        const iomb_view view = to_view(source);
        check_status(iomb_gather(&view, staging, stream));
        check_cuda("cudaMemcpyAsync(D2H)",
                   cudaMemcpyAsync(destination.data(), staging, destination.size(),
                                   cudaMemcpyDeviceToHost, stream));
        drain_transfer_stream(stream);
    }

    B200Device& device_;
    void* address_ = nullptr;
};

std::unique_ptr<Tensor> B200Device::create_tensor(const TensorSpec& spec) {
    return std::make_unique<B200Tensor>(spec, *this);
}

// ---- operation queue ----------------------------------------------------------

constexpr std::size_t kMaxOwners = 8;
constexpr std::size_t kMaxLeases = 2;
constexpr std::uint32_t kCaptureCells = 64;   // embedding status cells recordings may use

struct OwnerList {
    std::array<detail::BinaryOwnerRegistration, kMaxOwners> owners{};
    std::size_t count = 0;
    void add(const TensorView& view) {
        owners[count++] = detail::BinaryOwnerRegistration{
                view.owner_identity(), const_cast<void*>(view.native_handle())};
    }
    // A workspace range several operations in flight may read at once (control words):
    // registered like a tensor owner rather than leased exclusively.
    void add(const RawWorkspaceView& workspace) {
        owners[count++] = detail::BinaryOwnerRegistration{
                workspace.owner_identity(), detail::WorkspaceValidation::address(workspace)};
    }
};

// Entry ids of one submission: plain data, so a retirement record can carry them.
struct EntryList {
    std::array<detail::EntryId, kMaxOwners> ids{};
    std::uint32_t count = 0;
};

// register_binary_entries (include/iom/detail/workspace_registry.hpp:142-178) for up to
// six owners: one registry entry per distinct owner, all or nothing.
EntryList register_owners(detail::RegistryState& state, detail::QueueId queue_id,
                          std::uint64_t sequence, const OwnerList& owners,
                          const detail::Fence& fence) {
    std::lock_guard<std::mutex> lock(state.allocation_mutex);
    EntryList result;
    try {
        for (std::size_t index = 0; index < owners.count; ++index) {
            const detail::BinaryOwnerRegistration owner = owners.owners[index];
            if (owner.identity == nullptr || owner.address == nullptr) {
                throw std::invalid_argument("operation owner identity or address is null");
            }
            bool duplicate = false;
            for (std::size_t prior = 0; prior < index; ++prior) {
                if (owners.owners[prior].identity == owner.identity) duplicate = true;
            }
            if (duplicate) continue;
            const detail::EntryId id = detail::allocate_registry_id(state.next_entry_id);
            state.registry.register_entry(id, owner.address, sequence, queue_id,
                                          detail::Fence(fence));
            result.ids[result.count++] = id;
        }
    } catch (...) {
        if (result.count != 0) {
            state.registry.remove_entries(
                    std::span<const detail::EntryId>(result.ids.data(), result.count));
        }
        throw;
    }
    return result;
}

}  // namespace

namespace b200 {
// A recorded sequence: the instantiated graph and the status cells its embeddings write.
class CapturedSequence {
public:
    ~CapturedSequence() {
        if (exec != nullptr) (void)cudaGraphExecDestroy(exec);
        if (graph != nullptr) (void)cudaGraphDestroy(graph);
    }
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    const void* queue = nullptr;
    std::uint32_t first_cell = 0;
    std::uint32_t cell_count = 0;
};
}  // namespace b200

namespace {

class B200Queue final : public DeviceOps {
    enum class Proof : std::uint8_t { event, drained, unknown };

    // One accepted, launched operation waiting for its completion proof. Plain data.
    struct Retirement {
        std::uint64_t sequence = 0;
        std::uint32_t event_slot = 0;
        Proof proof = Proof::event;
        bool has_status = false;            // embedding: the slot's pinned status cell
        bool launch_failed = false;         // the native step threw: slot_failures_[event_slot]
        std::uint32_t capture_first = 0;    // replay: status cells of the recording
        std::uint32_t capture_count = 0;
        EntryList entries;
        std::array<detail::WorkspaceLease, kMaxLeases> leases{};
        std::uint32_t lease_count = 0;
    };

public:
    explicit B200Queue(B200Device& device)
            : DeviceOps(device), device_(&device),
              registry_queue_id_(detail::allocate_queue_id(device.registry_state())) {
        device_->activate();
        check_cuda("cudaStreamCreate", cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
        // One event per in-flight credit, one more so that an acquisition never waits for
        // the retirement that is just running; one pinned status cell per event, plus the
        // cells recordings use.
        const std::size_t slots = device.queue_config().max_in_flight_per_queue + 1;
        try {
            events_.resize(slots, nullptr);
            for (cudaEvent_t& event : events_) {
                check_cuda("cudaEventCreate",
                           cudaEventCreateWithFlags(&event, cudaEventDisableTiming));
            }
            slot_failures_.resize(slots);
            free_slots_.reserve(slots);
            for (std::size_t i = slots; i-- > 0;) free_slots_.push_back(static_cast<std::uint32_t>(i));
            ring_.resize(slots + 1);
            check_cuda("cudaMallocHost",
                       cudaMallocHost(reinterpret_cast<void**>(&status_cells_),
                                      (slots + kCaptureCells) * sizeof(std::uint32_t)));
            capture_cells_ = status_cells_ + slots;
        } catch (...) {
            destroy_native();
            throw;
        }
        worker_ = std::thread([this] { run_worker(); });
    }

    ~B200Queue() override {
        close_and_drain();
        {
            std::lock_guard<std::mutex> lock(publish_mutex_);
            shutdown_.store(true, std::memory_order_release);
            published_.fetch_add(1, std::memory_order_release);   // wakes the worker
        }
        published_.notify_all();
        if (worker_.joinable()) worker_.join();
        device_->registry_state().registry.invalidate_entries_for_queue(registry_queue_id_);
        destroy_native();
    }

    [[nodiscard]] cudaStream_t stream() const noexcept { return stream_; }
    [[nodiscard]] std::size_t quarantined_events() const noexcept {
        return quarantined_events_.load(std::memory_order_acquire);
    }

    // ---- extensions (see iom_b200_backend.hpp) --------------------------------------

    // One admission / registration / submission / failure-mapping path for the entries
    // outside the facade: the views' owners are registered and the workspace ranges
    // leased in the prepare step, released by the retirement, rolled back on failure.
    template <typename Launch>
    oid extension(std::initializer_list<const TensorView*> views,
                  std::initializer_list<RawWorkspaceView> workspaces, Launch launch,
                  std::initializer_list<RawWorkspaceView> shared = {}) noexcept {
        try {
            validate_views(queue_device(), views);
            if (workspaces.size() > kMaxLeases) throw std::invalid_argument("too many workspaces");
            struct Prepared {
                OwnerList owners;
                std::vector<RawWorkspaceView> workspaces;   // views copy but do not assign
                EntryList entries;
                std::array<detail::WorkspaceLease, kMaxLeases> leases{};
                std::uint32_t lease_count = 0;
            };
            auto prepared = std::make_shared<Prepared>();
            std::vector<TensorView> operands;
            operands.reserve(views.size());
            for (const TensorView* view : views) {
                prepared->owners.add(*view);
                operands.push_back(*view);
            }
            for (const RawWorkspaceView& workspace : workspaces) {
                (void)detail::WorkspaceValidation::validated(
                        queue_device(), workspace, workspace.empty() ? 1 : workspace.byte_size(), 32,
                        std::span<const TensorView>(operands.data(), operands.size()));
                prepared->workspaces.push_back(workspace);
            }
            for (const RawWorkspaceView& workspace : shared) {
                (void)detail::WorkspaceValidation::validated(
                        queue_device(), workspace, workspace.empty() ? 1 : workspace.byte_size(), 32,
                        std::span<const TensorView>(operands.data(), operands.size()));
                prepared->owners.add(workspace);
            }
            check_pre_acceptance_faults();
            detail::RegistryState& state = device_->registry_state();
            auto undo = [prepared, &state] {
                if (prepared->entries.count != 0) {
                    state.registry.remove_entries(std::span<const detail::EntryId>(
                            prepared->entries.ids.data(), prepared->entries.count));
                    prepared->entries = {};
                }
                for (std::uint32_t i = 0; i < prepared->lease_count; ++i) {
                    detail::complete_workspace_lease(state, prepared->leases[i], true);
                }
                prepared->lease_count = 0;
            };
            std::lock_guard<std::mutex> order(submission_order_mutex_);
            return submit_prepared(
                    [this, prepared, &state, undo](std::uint64_t sequence) {
                        const detail::Fence proof = fence();
                        try {
                            for (const RawWorkspaceView& workspace : prepared->workspaces) {
                                prepared->leases[prepared->lease_count] =
                                        detail::acquire_workspace_lease(
                                                state, workspace.owner_identity(),
                                                detail::WorkspaceValidation::address(workspace),
                                                workspace.byte_size(), sequence,
                                                registry_queue_id_, proof);
                                ++prepared->lease_count;
                            }
                            prepared->entries = register_owners(state, registry_queue_id_, sequence,
                                                                prepared->owners, proof);
                        } catch (...) {
                            undo();
                            throw;
                        }
                    },
                    [this, prepared, launch](std::uint64_t sequence) {
                        const std::uint32_t slot = acquire_event_slot();
                        Retirement record;
                        try {
                            device_->activate();
                            inject_launch_fault();
                            check_status(launch(stream_));
                        } catch (...) {
                            // The operation is accepted: its failure is retained and
                            // rethrown by every wait (src/shared/gpu_queue_operations.inl:1030-1056).
                            slot_failures_[slot] = std::current_exception();
                            record.launch_failed = true;
                        }
                        record.entries = prepared->entries;
                        record.leases = prepared->leases;
                        record.lease_count = prepared->lease_count;
                        retire(sequence, slot, record);
                    },
                    undo);
        } catch (...) {
            return map_exception(std::current_exception());
        }
    }

    oid add_rmsnorm(const TensorView& x, const TensorView& residual, const TensorView& scale,
                    TensorView& sum, TensorView& out, float eps) noexcept {
        const iomb_view vx = to_view(x), vr = to_view(residual), vw = to_view(scale),
                        vs = to_view(sum), vo = to_view(out);
        const int order = facade_order(x.spec().data_type);
        return extension({&x, &residual, &scale, &sum, &out}, {},
                         [vx, vr, vw, vs, vo, eps, order](cudaStream_t stream) {
                             return iomb_add_rmsnorm(&vx, &vr, &vw, &vs, &vo, eps, order, stream);
                         });
    }

    oid silu_mul(const TensorView& x, const TensorView& up, TensorView* activated,
                 TensorView& out) noexcept {
        const iomb_view vx = to_view(x), vu = to_view(up), vo = to_view(out);
        if (activated != nullptr) {
            const iomb_view va = to_view(*activated);
            return extension({&x, &up, activated, &out}, {}, [vx, vu, va, vo](cudaStream_t stream) {
                return iomb_silu_mul(&vx, &vu, &va, &vo, stream);
            });
        }
        return extension({&x, &up, &out}, {}, [vx, vu, vo](cudaStream_t stream) {
            return iomb_silu_mul(&vx, &vu, nullptr, &vo, stream);
        });
    }

    oid cast(const TensorView& source, TensorView& destination) noexcept {
        const iomb_view vs = to_view(source), vd = to_view(destination);
        return extension({&source, &destination}, {},
                         [vs, vd](cudaStream_t stream) { return iomb_cast(&vs, &vd, stream); });
    }

    oid cache_append_batched(const TensorView& source, TensorView& destination,
                             RawWorkspaceView control) noexcept {
        const std::size_t sequences = source.spec().shape.dimensions()[0];
        if (control.byte_size() < b200::batched_control_bytes(sequences)) {
            return to_oid(OidError::InvalidArgument);
        }
        const iomb_view vs = to_view(source), vd = to_view(destination);
        auto* words = static_cast<std::uint32_t*>(detail::WorkspaceValidation::address(control));
        // The control range is registered, not leased: the K and V appends of every layer
        // of a step share one range of offsets, and the queue runs them in order.
        return extension({&source, &destination}, {}, [vs, vd, words](cudaStream_t stream) {
            return iomb_cache_append_batched(&vs, &vd, words + 8, words, stream);
        }, {control});
    }

    oid sumsq(const TensorView& x, RawWorkspaceView workspace) noexcept {
        if (workspace.byte_size() < b200::sumsq_workspace_bytes()) {
            return to_oid(OidError::InvalidArgument);
        }
        const iomb_view vx = to_view(x);
        auto* base = static_cast<unsigned char*>(detail::WorkspaceValidation::address(workspace));
        return extension({&x}, {workspace}, [vx, base](cudaStream_t stream) {
            return iomb_sumsq(&vx, base + 32, reinterpret_cast<float*>(base), stream);
        });
    }

    // stage: 0 scale/mask, 1 softmax, 2 both (scores only read), 3 both (scaled scores stored)
    oid sdpa_stage(int stage, const b200::SdpaStages& s, RawWorkspaceView workspace) noexcept {
        const iomb_sdpa_stages request{s.scores, s.probability, s.planes, s.Hq, s.Hkv,
                                       s.R, s.C, s.D, s.a, s.L};
        return extension({}, {workspace}, [stage, request](cudaStream_t stream) {
            switch (stage) {
                case 0: return iomb_sdpa_scale_mask(&request, stream);
                case 1: return iomb_sdpa_softmax(&request, stream);
                default: return iomb_sdpa_scale_mask_softmax(&request, stage == 3 ? 1 : 0, stream);
            }
        });
    }

    oid sdpa_canonicalize_output(TensorView& out) noexcept {
        const iomb_view vo = to_view(out);
        return extension({&out}, {}, [vo](cudaStream_t stream) {
            return iomb_sdpa_canonicalize_output(&vo, stream);
        });
    }

    // ---- recording and replay ------------------------------------------------------

    void capture_begin() {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        if (capturing_) throw std::logic_error("the queue is already recording");
        device_->activate();
        // Everything issued before must have retired: a recording holds no events.
        check_cuda("cudaStreamSynchronize", cudaStreamSynchronize(stream_));
        check_cuda("cudaStreamBeginCapture",
                   cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
        capturing_ = true;
        capture_first_cell_ = next_capture_cell_;
    }

    std::shared_ptr<b200::CapturedSequence> capture_end() {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        if (!capturing_) throw std::logic_error("the queue is not recording");
        capturing_ = false;
        device_->activate();
        auto recorded = std::make_shared<b200::CapturedSequence>();
        check_cuda("cudaStreamEndCapture", cudaStreamEndCapture(stream_, &recorded->graph));
        check_cuda("cudaGraphInstantiate", cudaGraphInstantiate(&recorded->exec, recorded->graph, 0));
        recorded->queue = this;
        recorded->first_cell = capture_first_cell_;
        recorded->cell_count = next_capture_cell_ - capture_first_cell_;
        return recorded;
    }

    oid replay(const std::shared_ptr<b200::CapturedSequence>& recorded) noexcept {
        try {
            if (recorded == nullptr || recorded->queue != this || recorded->exec == nullptr) {
                throw std::invalid_argument("the recording does not belong to this queue");
            }
            std::lock_guard<std::mutex> order(submission_order_mutex_);
            if (capturing_) throw std::logic_error("a recording cannot be replayed while recording");
            return submit([this, recorded](std::uint64_t sequence) {
                const std::uint32_t slot = acquire_event_slot();
                Retirement record;
                try {
                    device_->activate();
                    inject_launch_fault();
                    for (std::uint32_t i = 0; i < recorded->cell_count; ++i) {
                        capture_cells_[recorded->first_cell + i] = 0;
                    }
                    check_cuda("cudaGraphLaunch", cudaGraphLaunch(recorded->exec, stream_));
                } catch (...) {
                    slot_failures_[slot] = std::current_exception();
                    record.launch_failed = true;
                }
                record.capture_first = recorded->first_cell;
                record.capture_count = recorded->cell_count;
                retire(sequence, slot, record);
            });
        } catch (...) {
            return map_exception(std::current_exception());
        }
    }

protected:
    [[nodiscard]] std::string_view backend_label() const noexcept override { return "B200"; }

    oid copy_impl(const TensorView& source, TensorView& destination) override {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        check_pre_acceptance_faults();
        return submit_copy(
                source, destination, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const CopyRequest& request,
                       detail::EntryRegistration entries) {
                    EntryList list;
                    list.ids[0] = entries.source;
                    list.ids[1] = entries.destination;
                    list.count = 2;
                    launch_and_retire(sequence, list, {}, [&] {
                        if (request.no_op) return;
                        const iomb_view src = to_view(request.source);
                        const iomb_view dst = to_view(request.destination);
                        check_status(iomb_copy(&src, &dst, stream_));
                    });
                });
    }

    static_assert(static_cast<int>(BinaryOperation::Add) == IOMB_ADD
                          && static_cast<int>(BinaryOperation::Mul) == IOMB_MUL
                          && static_cast<int>(BinaryOperation::Sub) == IOMB_SUB
                          && static_cast<int>(BinaryOperation::Div) == IOMB_DIV,
                  "BinaryOperation and iomb_binary_op must share their ordinals");

    oid binary_impl(const BinaryRequest& request) override {
        if (iomb_binary_supported(static_cast<std::uint32_t>(request.out.spec.data_type)) == 0) {
            throw detail::UnsupportedOperation();
        }
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        check_pre_acceptance_faults();
        return submit_binary(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const BinaryRequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    launch_and_retire(sequence, to_list(entries), captured.workspace_lease, [&] {
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
        check_pre_acceptance_faults();
        return submit_rmsnorm(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const RmsnormRequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    launch_and_retire(sequence, to_list(entries), {}, [&] {
                        const iomb_view x = to_view(captured.x), w = to_view(captured.scale),
                                        out = to_view(captured.out);
                        check_status(iomb_rmsnorm(&x, &w, &out, captured.epsilon,
                                                  facade_order(captured.x.spec.data_type), stream_));
                    });
                });
    }

    [[nodiscard]] WorkspaceRequirements embedding_workspace_requirements_impl(
            const TensorView&, const TensorView&, const TensorView&) override {
        // First u32 of the range is the status word (0 ok / 1 invalid id),
        // docs/BACKEND_CONTRACT/embedding-lookup.md:178-209.
        return {32, 32};
    }

    oid embedding_impl(const EmbeddingRequest& request) override {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        check_pre_acceptance_faults();
        return submit_embedding(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const EmbeddingRequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    auto* status = static_cast<std::uint32_t*>(
                            detail::WorkspaceValidation::address(captured.workspace));
                    launch_and_retire(
                            sequence, to_list(entries), captured.workspace_lease,
                            [&] {
                                const iomb_view table = to_view(captured.table),
                                                ids = to_view(captured.indices),
                                                out = to_view(captured.out);
                                check_status(iomb_embedding(&table, &ids, &out, status, stream_));
                            },
                            status);
                });
    }

    [[nodiscard]] WorkspaceRequirements cache_append_workspace_requirements(
            const CacheAppendRequest& request) override {
        (void)request;   // every leaf width (8..64 bits, and 2, 4, 6 bits) has a kernel
        return {0, 1};
    }

    oid cache_append_impl(const CacheAppendRequest& request) override {
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        check_pre_acceptance_faults();
        return submit_cache_append(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const CacheAppendRequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    launch_and_retire(sequence, to_list(entries), captured.workspace_lease, [&] {
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
        check_pre_acceptance_faults();
        return submit_silu(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this](std::uint64_t sequence, const SiLURequest& captured,
                       detail::BinaryEntryRegistration entries) {
                    launch_and_retire(sequence, to_list(entries), {}, [&] {
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
        // A table that is not yet resident is placed in the region reserved at device
        // construction (no allocation); a full region refuses the request.
        const std::size_t rows = request.x.dimensions[request.x.rank - 2];
        const std::size_t width = request.x.dimensions[request.x.rank - 1];
        const float* table = device_->rope_table(request.theta, width, request.a + rows);
        const float* first = table + request.a * (width / 2) * 2;
        std::lock_guard<std::mutex> order(submission_order_mutex_);
        check_pre_acceptance_faults();
        return submit_rope(
                request, device_->registry_state(), registry_queue_id_, fence(),
                [this, first](std::uint64_t sequence, const RopeRequest& captured,
                              detail::BinaryEntryRegistration entries) {
                    launch_and_retire(sequence, to_list(entries), {}, [&] {
                        const iomb_view x = to_view_fixed(captured.x), out = to_view_fixed(captured.out);
                        check_status(iomb_rope(&x, &out, captured.a, first, stream_));
                    });
                });
    }

private:
    static EntryList to_list(const detail::BinaryEntryRegistration& entries) {
        EntryList list;
        for (std::size_t i = 0; i < entries.count; ++i) list.ids[i] = entries.entries[i];
        list.count = static_cast<std::uint32_t>(entries.count);
        return list;
    }

    static oid map_exception(std::exception_ptr failure) noexcept {
        try {
            std::rethrow_exception(failure);
        } catch (const detail::UnsupportedOperation&) {
            return to_oid(OidError::Unsupported);
        } catch (const std::bad_alloc&) {
            return to_oid(OidError::ResourceExhausted);
        } catch (const std::overflow_error&) {
            return to_oid(OidError::Overflow);
        } catch (const std::invalid_argument&) {
            return to_oid(OidError::InvalidArgument);
        } catch (const std::exception&) {
            return to_oid(OidError::DeviceError);
        } catch (...) {
            return to_oid(OidError::InternalError);
        }
    }

    // Host registration / preparation faults are consumed before common acceptance
    // reserves a sequence (src/shared/gpu_queue_operations.inl:8-13).
    static void check_pre_acceptance_faults() {
        if (consume_fault(b200::SubmissionFault::registration)
                || consume_fault(b200::SubmissionFault::outcome_insertion)) {
            throw std::bad_alloc();
        }
    }

    static void inject_launch_fault() {
        if (consume_fault(b200::SubmissionFault::launch)) {
            throw std::runtime_error("kernel launch: injected failure");
        }
    }

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

    // An event of the fixed set. None free (all in flight or quarantined): the node stays
    // parked and is retried when a retirement returns one (include/iom/iom.hpp:32-40).
    std::uint32_t acquire_event_slot() {
        std::lock_guard<std::mutex> lock(slot_mutex_);
        if (free_slots_.empty()) throw detail::AdmissionResourceUnavailable{};
        const std::uint32_t slot = free_slots_.back();
        free_slots_.pop_back();
        return slot;
    }
    void release_event_slot(std::uint32_t slot) noexcept {
        std::lock_guard<std::mutex> lock(slot_mutex_);
        free_slots_.push_back(slot);      // capacity reserved at construction
    }

    // Launches through `launch`, then retires. The operation has been accepted by the time
    // this runs, so a failing native step is a retained failure: the token completes with
    // the exception and every wait rethrows it (src/shared/gpu_queue_operations.inl:1030-1056).
    // Only the lack of a free event leaves the node parked.
    template <typename Launch>
    void launch_and_retire(std::uint64_t sequence, const EntryList& entries,
                           detail::WorkspaceLease lease, Launch&& launch,
                           std::uint32_t* device_status = nullptr) {
        const std::uint32_t slot = acquire_event_slot();
        Retirement record;
        try {
            device_->activate();
            inject_launch_fault();
            launch();
            if (device_status != nullptr) {
                // The status word goes to a pinned cell on the same stream: the slot's own
                // cell, or a cell of the recording when one is being made.
                std::uint32_t* cell = status_cells_ + slot;
                if (capturing_) {
                    if (next_capture_cell_ >= kCaptureCells) throw std::bad_alloc();
                    cell = capture_cells_ + next_capture_cell_++;
                }
                *cell = 0;
                cudaError_t copied = cudaMemcpyAsync(cell, device_status, sizeof(std::uint32_t),
                                                     cudaMemcpyDeviceToHost, stream_);
                if (consume_fault(b200::SubmissionFault::embedding_status_copy)) {
                    copied = cudaErrorInvalidValue;
                }
                if (copied != cudaSuccess) {
                    // The kernel is in flight: let it finish before the failure is reported.
                    if (!capturing_) (void)cudaStreamSynchronize(stream_);
                    check_cuda("cudaMemcpyAsync(status)", copied);
                }
                record.has_status = !capturing_;
            }
        } catch (...) {
            slot_failures_[slot] = std::current_exception();
            record.launch_failed = true;
            record.has_status = false;
        }
        record.entries = entries;
        if (lease.entry_id != 0) {
            record.leases[0] = lease;
            record.lease_count = 1;
        }
        retire(sequence, slot, record);
    }

    // Obtains the completion proof and hands the record to the worker. While recording
    // there is nothing to wait for: the operation is retired on the spot.
    void retire(std::uint64_t sequence, std::uint32_t slot, Retirement record) noexcept {
        record.sequence = sequence;
        record.event_slot = slot;
        if (capturing_) {
            std::exception_ptr failure;
            if (record.launch_failed) failure = std::move(slot_failures_[slot]);
            release_event_slot(slot);
            finish(record, true, std::move(failure));
            return;
        }
        bool recorded = false;
        for (int attempt = 0; attempt < 2 && !recorded; ++attempt) {
            cudaError_t status = cudaEventRecord(events_[slot], stream_);
            if (consume_fault(b200::SubmissionFault::event_record)) status = cudaErrorInvalidValue;
            recorded = status == cudaSuccess;
        }
        if (recorded) {
            record.proof = Proof::event;
        } else {
            (void)cudaGetLastError();
            const cudaError_t drained = cudaStreamSynchronize(stream_);
            const bool injected = consume_fault(b200::SubmissionFault::stream_synchronize);
            record.proof = drained == cudaSuccess && !injected ? Proof::drained : Proof::unknown;
        }
        {
            // Producers are the submitting thread and, for parked nodes, the worker
            // (through complete -> pump_admission); the facade runs one at a time.
            std::lock_guard<std::mutex> lock(publish_mutex_);
            const std::uint64_t index = published_.load(std::memory_order_relaxed);
            ring_[index % ring_.size()] = record;
            published_.store(index + 1, std::memory_order_release);
        }
        published_.notify_one();
    }

    // Releases what the operation held and completes its sequence.
    void finish(const Retirement& record, bool proven, std::exception_ptr failure) noexcept {
        detail::RegistryState& state = device_->registry_state();
        const std::span<const detail::EntryId> ids(record.entries.ids.data(), record.entries.count);
        if (failure != nullptr || !proven) {
            state.registry.invalidate_entries(ids);
        } else {
            for (const detail::EntryId id : ids) (void)state.registry.try_release_entry(id);
        }
        for (std::uint32_t i = 0; i < record.lease_count; ++i) {
            detail::complete_workspace_lease(state, record.leases[i], proven);
        }
        try {
            complete(record.sequence, std::move(failure));
        } catch (...) {
        }
    }

    void run_worker() noexcept {
        (void)cudaSetDevice(static_cast<int>(device_->backend_device()));
        std::uint64_t consumed = 0;
        std::uint64_t proven_count = 0;     // ring records known complete through a later event
        for (;;) {
            std::uint64_t available = published_.load(std::memory_order_acquire);
            while (available == consumed) {
                published_.wait(available, std::memory_order_acquire);
                available = published_.load(std::memory_order_acquire);
            }
            // The destructor bumps the counter once more after the last record.
            if (shutdown_.load(std::memory_order_acquire) && consumed + 1 == available) return;
            const Retirement record = ring_[consumed % ring_.size()];
            ++consumed;
            std::exception_ptr failure;
            bool proven = true;
            if (record.proof == Proof::event && consumed <= proven_count) {
                // A later operation of this stream has completed: so has this one.
            } else if (record.proof == Proof::event) {
                // The stream runs its operations in order, so a later event that has already
                // completed proves every record before it: when this thread is behind, one
                // query retires the whole backlog (the submitting thread shares the driver
                // with this one, and fewer blocking waits leave it more room). Otherwise the
                // record's own event is waited for, so no token completes later than its
                // operation.
                std::uint64_t newest = consumed - 1;
                for (std::uint64_t i = consumed; i < available; ++i) {
                    if (shutdown_.load(std::memory_order_acquire) && i + 1 == available) break;
                    if (ring_[i % ring_.size()].proof == Proof::event) newest = i;
                }
                cudaError_t status = cudaErrorNotReady;
                if (newest != consumed - 1) {
                    status = cudaEventQuery(events_[ring_[newest % ring_.size()].event_slot]);
                    if (status == cudaSuccess) proven_count = newest + 1;   // records [0, newest]
                    else (void)cudaGetLastError();
                }
                if (status != cudaSuccess) status = cudaEventSynchronize(events_[record.event_slot]);
                if (status != cudaSuccess) {
                    proven = false;
                    failure = std::make_exception_ptr(std::runtime_error(
                            std::string("B200 operation failed: ") + cudaGetErrorString(status)));
                }
            } else if (record.proof == Proof::unknown) {
                proven = false;
                failure = std::make_exception_ptr(std::runtime_error(
                        "B200 operation: completion could not be proven"));
            }
            if (record.launch_failed) {
                std::exception_ptr retained = std::move(slot_failures_[record.event_slot]);
                slot_failures_[record.event_slot] = nullptr;
                if (failure == nullptr) failure = std::move(retained);
            }
            if (proven && failure == nullptr) {
                bool invalid_id = record.has_status && status_cells_[record.event_slot] != 0;
                for (std::uint32_t i = 0; i < record.capture_count; ++i) {
                    if (capture_cells_[record.capture_first + i] != 0) invalid_id = true;
                }
                if (invalid_id) {
                    // An invalid id is a retained invalid_argument
                    // (src/shared/gpu_queue_operations.inl:1080-1095).
                    failure = std::make_exception_ptr(
                            std::invalid_argument("embedding index is negative or out of range"));
                }
            }
            // An event whose completion is unknown is never handed out again
            // (src/shared/event_ring.hpp:220-232).
            if (proven) {
                release_event_slot(record.event_slot);
            } else {
                quarantined_events_.fetch_add(1, std::memory_order_acq_rel);
            }
            finish(record, proven, std::move(failure));
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
    std::vector<std::uint32_t> free_slots_;
    std::vector<std::exception_ptr> slot_failures_;   // one per event, set before publication
    std::mutex slot_mutex_;
    std::uint32_t* status_cells_ = nullptr;
    std::uint32_t* capture_cells_ = nullptr;
    std::uint32_t next_capture_cell_ = 0;
    std::uint32_t capture_first_cell_ = 0;
    bool capturing_ = false;
    std::mutex submission_order_mutex_;
    std::vector<Retirement> ring_;
    std::mutex publish_mutex_;
    std::atomic<std::uint64_t> published_{0};
    std::atomic<bool> shutdown_{false};
    std::atomic<std::size_t> quarantined_events_{0};
    std::thread worker_;
};

std::unique_ptr<DeviceOps> B200Device::create_ops() {
    return std::make_unique<B200Queue>(*this);
}

B200Queue* native_queue(DeviceOps& queue) noexcept { return dynamic_cast<B200Queue*>(&queue); }

}  // namespace

std::unique_ptr<Device> make_b200_device(
        std::uint32_t ordinal, DeviceMemoryConfig memory_config, QueueConfig queue_config,
        b200::Options options) {
    return std::make_unique<B200Device>(ordinal, memory_config, queue_config, options);
}

namespace b200 {

oid add_rmsnorm(DeviceOps& queue, const TensorView& x, const TensorView& residual,
                const TensorView& scale, TensorView& sum, TensorView& out, float eps) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->add_rmsnorm(x, residual, scale, sum, out, eps);
}

oid silu_mul(DeviceOps& queue, const TensorView& x, const TensorView& up, TensorView* activated,
             TensorView& out) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->silu_mul(x, up, activated, out);
}

oid cast(DeviceOps& queue, const TensorView& source, TensorView& destination) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->cast(source, destination);
}

oid cache_append_batched(DeviceOps& queue, const TensorView& source, TensorView& destination,
                         RawWorkspaceView control) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->cache_append_batched(source, destination, control);
}

std::size_t batched_control_bytes(std::size_t sequences) {
    return (32 + sequences * sizeof(std::uint32_t) + 31) / 32 * 32;
}

oid sumsq(DeviceOps& queue, const TensorView& x, RawWorkspaceView workspace) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->sumsq(x, workspace);
}

std::size_t sumsq_workspace_bytes() {
    return 32 + static_cast<std::size_t>(iomb_sumsq_scratch_bytes());
}

oid sdpa_scale_mask(DeviceOps& queue, const SdpaStages& stages, RawWorkspaceView workspace) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->sdpa_stage(0, stages, workspace);
}
oid sdpa_softmax(DeviceOps& queue, const SdpaStages& stages, RawWorkspaceView workspace) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->sdpa_stage(1, stages, workspace);
}
oid sdpa_scale_mask_softmax(DeviceOps& queue, const SdpaStages& stages, bool keep_scores,
                            RawWorkspaceView workspace) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->sdpa_stage(keep_scores ? 3 : 2, stages, workspace);
}
oid sdpa_canonicalize_output(DeviceOps& queue, TensorView& out) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->sdpa_canonicalize_output(out);
}

void capture_begin(DeviceOps& queue) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) throw std::invalid_argument("not a B200 queue");
    native->capture_begin();
}

std::shared_ptr<CapturedSequence> capture_end(DeviceOps& queue) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) throw std::invalid_argument("not a B200 queue");
    return native->capture_end();
}

oid replay(DeviceOps& queue, const std::shared_ptr<CapturedSequence>& sequence) {
    B200Queue* native = native_queue(queue);
    if (native == nullptr) return to_oid(OidError::InvalidArgument);
    return native->replay(sequence);
}

void* native_stream(DeviceOps& queue) {
    B200Queue* native = native_queue(queue);
    return native == nullptr ? nullptr : static_cast<void*>(native->stream());
}

void inject_submission_fault_for_testing(SubmissionFault fault) noexcept {
    // event_record: the record and its retry fail, and so does the drain that would
    // prove completion otherwise (src/cuda/copy.cu:728-737).
    g_event_record_failures.store(fault == SubmissionFault::event_record ? 2 : 0,
                                  std::memory_order_release);
    g_stream_sync_failures.store(
            fault == SubmissionFault::event_record || fault == SubmissionFault::stream_synchronize
                    ? 1 : 0,
            std::memory_order_release);
    const bool counted = fault == SubmissionFault::event_record
            || fault == SubmissionFault::stream_synchronize;
    g_fault.store(counted ? SubmissionFault::none : fault, std::memory_order_release);
}

std::size_t quarantined_event_count(DeviceOps& queue) {
    B200Queue* native = native_queue(queue);
    return native == nullptr ? 0 : native->quarantined_events();
}

}  // namespace b200
}  // namespace iom
