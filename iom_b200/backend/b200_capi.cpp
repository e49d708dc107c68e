// C driver interface of the B200 backend (include/iom_b200_backend_c.h): handles over
// iom::Device / Tensor / TensorView / DeviceOps of a device from make_b200_device, and a
// small program runner that issues facade operations from C++ (no interpreter between two
// submissions) and times them on the queue's stream.
#include "iom_b200_backend_c.h"

#include <cuda_runtime_api.h>

#include <chrono>
#include <deque>
#include <cstddef>
#include <exception>
#include <memory>
#include <new>
#include <span>
#include <stdexcept>
#include <string>
#include <vector>

#include "iom_b200_backend.hpp"

namespace {

thread_local std::string g_error;

struct DeviceBox {
    std::unique_ptr<iom::Device> device;
};
struct TensorBox {
    std::unique_ptr<iom::Tensor> tensor;
};
struct WorkspaceBox {
    std::unique_ptr<iom::RawWorkspace> workspace;
};
struct ViewBox {
    iom::TensorView view;
};
struct QueueBox {
    std::unique_ptr<iom::DeviceOps> ops;
    std::size_t credits = 1;      // operations the queue keeps in flight before it parks one
    int ordinal = 0;              // the device's CUDA ordinal (the runner's own events live there)
};

int classify(std::exception_ptr failure) {
    try {
        std::rethrow_exception(failure);
    } catch (const std::invalid_argument& e) {
        g_error = e.what();
        return 1;
    } catch (const std::out_of_range& e) {
        g_error = e.what();
        return 2;
    } catch (const std::overflow_error& e) {
        g_error = e.what();
        return 3;
    } catch (const std::bad_alloc& e) {
        g_error = e.what();
        return 4;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 5;
    } catch (...) {
        g_error = "unknown exception";
        return 6;
    }
}

template <typename Body>
void* guarded(Body&& body) {
    try {
        return body();
    } catch (...) {
        (void)classify(std::current_exception());
        return nullptr;
    }
}

iom::TensorView& view_of(void* handle) {
    if (handle == nullptr) throw std::invalid_argument("operation names a null view");
    return static_cast<ViewBox*>(handle)->view;
}

iom::RawWorkspaceView workspace_of(void* handle) {
    if (handle == nullptr) return {};
    return static_cast<WorkspaceBox*>(handle)->workspace->view();
}

// Issues one operation; returns its oid (0 for the synchronous host transfers).
iom::oid issue(iom::DeviceOps& ops, const iomb_backend_op& op) {
    void* const* v = op.views;
    switch (op.opcode) {
        case IOMB_BACKEND_ADD: return ops.add(view_of(v[0]), view_of(v[1]), view_of(v[2]));
        case IOMB_BACKEND_MUL: return ops.mul(view_of(v[0]), view_of(v[1]), view_of(v[2]));
        case IOMB_BACKEND_SUB: return ops.sub(view_of(v[0]), view_of(v[1]), view_of(v[2]));
        case IOMB_BACKEND_DIV: return ops.div(view_of(v[0]), view_of(v[1]), view_of(v[2]));
        case IOMB_BACKEND_RMSNORM:
            return ops.rmsnorm(view_of(v[0]), view_of(v[1]), view_of(v[2]), op.eps);
        case IOMB_BACKEND_ADD_RMSNORM:
            return iom::b200::add_rmsnorm(ops, view_of(v[0]), view_of(v[1]), view_of(v[2]),
                                          view_of(v[3]), view_of(v[4]), op.eps);
        case IOMB_BACKEND_COPY: return ops.copy(view_of(v[0]), view_of(v[1]));
        case IOMB_BACKEND_EMBEDDING:
            return ops.embedding(view_of(v[0]), view_of(v[1]), view_of(v[2]), workspace_of(op.workspace));
        case IOMB_BACKEND_CACHE_APPEND:
            return ops.cache_append(view_of(v[0]), view_of(v[1]), op.a);
        case IOMB_BACKEND_CACHE_APPEND_BATCHED:
            return iom::b200::cache_append_batched(ops, view_of(v[0]), view_of(v[1]),
                                                   workspace_of(op.workspace));
        case IOMB_BACKEND_SILU: return ops.silu(view_of(v[0]), view_of(v[1]));
        case IOMB_BACKEND_SILU_MUL:
            return iom::b200::silu_mul(ops, view_of(v[0]), view_of(v[1]), nullptr, view_of(v[2]));
        case IOMB_BACKEND_ROPE: return ops.rope(view_of(v[0]), view_of(v[1]), op.a, op.theta);
        case IOMB_BACKEND_CAST: return iom::b200::cast(ops, view_of(v[0]), view_of(v[1]));
        case IOMB_BACKEND_SUMSQ:
            return iom::b200::sumsq(ops, view_of(v[0]), workspace_of(op.workspace));
        case IOMB_BACKEND_FROM_HOST:
            view_of(v[0]).copy_from_host(
                    std::span<const std::byte>(static_cast<const std::byte*>(op.host), op.host_bytes),
                    workspace_of(op.workspace));
            return 0;
        case IOMB_BACKEND_TO_HOST:
            view_of(v[0]).copy_to_host(
                    std::span<std::byte>(static_cast<std::byte*>(op.host), op.host_bytes),
                    workspace_of(op.workspace));
            return 0;
        default: throw std::invalid_argument("unknown opcode");
    }
}

void check_cuda(const char* what, cudaError_t status) {
    if (status != cudaSuccess) {
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(status));
    }
}

}  // namespace

extern "C" {

const char* iomb_backend_last_error(void) { return g_error.c_str(); }

void* iomb_backend_device_create(uint32_t ordinal, uint64_t arena_bytes, uint32_t max_in_flight) {
    return guarded([&]() -> void* {
        auto box = std::make_unique<DeviceBox>();
        iom::QueueConfig queue_config{};
        if (max_in_flight != 0) queue_config.max_in_flight_per_queue = max_in_flight;
        box->device = iom::make_b200_device(ordinal, iom::DeviceMemoryConfig{arena_bytes}, queue_config);
        return box.release();
    });
}

void iomb_backend_device_destroy(void* device) { delete static_cast<DeviceBox*>(device); }

void* iomb_backend_queue_create(void* device) {
    return guarded([&]() -> void* {
        auto box = std::make_unique<QueueBox>();
        iom::Device& owner = *static_cast<DeviceBox*>(device)->device;
        box->ops = owner.create_ops();
        box->credits = owner.queue_config().max_in_flight_per_queue;
        box->ordinal = static_cast<int>(owner.backend_device());
        return box.release();
    });
}

void iomb_backend_queue_destroy(void* queue) { delete static_cast<QueueBox*>(queue); }

void* iomb_backend_tensor_create(void* device, const uint64_t* dims, uint32_t rank, uint32_t dtype) {
    return guarded([&]() -> void* {
        std::vector<std::size_t> shape(dims, dims + rank);
        const iom::TensorSpec spec{iom::TensorShape{std::move(shape)}, static_cast<iom::DataType>(dtype)};
        auto box = std::make_unique<TensorBox>();
        box->tensor = static_cast<DeviceBox*>(device)->device->create_tensor(spec);
        return box.release();
    });
}

void iomb_backend_tensor_destroy(void* tensor) { delete static_cast<TensorBox*>(tensor); }

void* iomb_backend_tensor_address(void* tensor) {
    return static_cast<TensorBox*>(tensor)->tensor->view().native_handle();
}

uint64_t iomb_backend_tensor_nbytes(void* tensor) {
    return static_cast<TensorBox*>(tensor)->tensor->view().spec().tiled_storage_nbytes();
}

void* iomb_backend_workspace_create(void* device, uint64_t bytes) {
    return guarded([&]() -> void* {
        auto box = std::make_unique<WorkspaceBox>();
        box->workspace = static_cast<DeviceBox*>(device)->device->create_workspace(bytes);
        return box.release();
    });
}

void iomb_backend_workspace_destroy(void* workspace) { delete static_cast<WorkspaceBox*>(workspace); }

void* iomb_backend_workspace_address(void* workspace) {
    return iom::detail::WorkspaceValidation::address(
            static_cast<WorkspaceBox*>(workspace)->workspace->view());
}

void* iomb_backend_view_full(void* tensor) {
    return guarded([&]() -> void* {
        return new ViewBox{static_cast<TensorBox*>(tensor)->tensor->view()};
    });
}

void* iomb_backend_view_select(void* view, uint64_t dim, uint64_t index) {
    return guarded([&]() -> void* { return new ViewBox{view_of(view).select(dim, index)}; });
}

void* iomb_backend_view_slice(void* view, uint64_t dim, uint64_t first, uint64_t count, uint64_t step) {
    return guarded([&]() -> void* { return new ViewBox{view_of(view).slice(dim, first, count, step)}; });
}

void iomb_backend_view_destroy(void* view) { delete static_cast<ViewBox*>(view); }

int iomb_backend_run(void* queue, const iomb_backend_op* operations, uint32_t count,
                     uint32_t warmup, uint32_t passes, uint32_t mode, iomb_backend_timing* timing) {
    cudaEvent_t start = nullptr, stop = nullptr;
    try {
        if (queue == nullptr || (operations == nullptr && count != 0) || timing == nullptr) {
            throw std::invalid_argument("iomb_backend_run: null argument");
        }
        iom::DeviceOps& ops = *static_cast<QueueBox*>(queue)->ops;
        // The current device is per host thread: a caller's worker thread starts on device 0.
        check_cuda("cudaSetDevice", cudaSetDevice(static_cast<QueueBox*>(queue)->ordinal));
        const cudaStream_t stream = static_cast<cudaStream_t>(iom::b200::native_stream(ops));
        if (stream == nullptr) throw std::invalid_argument("not a queue of the B200 backend");
        using clock = std::chrono::steady_clock;
        // Tokens not yet collected, oldest first. Never more than the queue's credits: an
        // operation beyond them would be accepted but parked and launched by a later
        // retirement, that is after the event that closes the timed region.
        const std::size_t credits = static_cast<QueueBox*>(queue)->credits;
        std::deque<iom::oid> tokens;
        double submit_seconds = 0.0;
        std::uint64_t issued = 0;
        auto wait_all = [&] {
            for (const iom::oid token : tokens) ops.wait(token);
            tokens.clear();
        };
        // One pass of the program, operation by operation.
        auto pass = [&](bool count_it) {
            for (uint32_t i = 0; i < count; ++i) {
                const iomb_backend_op& op = operations[i];
                if (op.opcode == IOMB_BACKEND_WAIT) {
                    wait_all();
                    continue;
                }
                while (tokens.size() >= credits) {
                    ops.wait(tokens.front());
                    tokens.pop_front();
                }
                const auto before = clock::now();
                const iom::oid token = issue(ops, op);
                if (count_it) {
                    submit_seconds += std::chrono::duration<double>(clock::now() - before).count();
                    ++issued;
                }
                if (token < 0) {
                    throw std::runtime_error("operation " + std::to_string(i) + " (opcode "
                                             + std::to_string(op.opcode) + ") was refused with oid "
                                             + std::to_string(token));
                }
                if (token > 0) {
                    if (mode == IOMB_BACKEND_WAIT_EACH) ops.wait(token);
                    else tokens.push_back(token);
                }
            }
        };
        std::shared_ptr<iom::b200::CapturedSequence> recording;
        if (mode == IOMB_BACKEND_RECORDED) {
            pass(false);            // once eagerly: one-time set-up must not be recorded
            wait_all();
            iom::b200::capture_begin(ops);
            try {
                pass(false);
            } catch (...) {
                try { (void)iom::b200::capture_end(ops); } catch (...) {}
                throw;
            }
            tokens.clear();         // tokens of recorded operations complete at once
            recording = iom::b200::capture_end(ops);
        }
        auto replay = [&](bool count_it) {
            const auto before = clock::now();
            const iom::oid token = iom::b200::replay(ops, recording);
            if (count_it) {
                submit_seconds += std::chrono::duration<double>(clock::now() - before).count();
                issued += 1;
            }
            if (token <= 0) throw std::runtime_error("replay was refused with oid " + std::to_string(token));
            while (tokens.size() >= credits) {
                ops.wait(tokens.front());
                tokens.pop_front();
            }
            tokens.push_back(token);
        };
        for (uint32_t i = 0; i < warmup; ++i) {
            if (recording) replay(false); else pass(false);
            wait_all();
        }
        check_cuda("cudaEventCreate", cudaEventCreate(&start));
        check_cuda("cudaEventCreate", cudaEventCreate(&stop));
        check_cuda("cudaStreamSynchronize", cudaStreamSynchronize(stream));
        const auto begin = clock::now();
        check_cuda("cudaEventRecord", cudaEventRecord(start, stream));
        for (uint32_t i = 0; i < passes; ++i) {
            if (recording) replay(true); else pass(true);
        }
        check_cuda("cudaEventRecord", cudaEventRecord(stop, stream));
        wait_all();
        check_cuda("cudaEventSynchronize", cudaEventSynchronize(stop));
        timing->host_seconds = std::chrono::duration<double>(clock::now() - begin).count();
        timing->submit_seconds = submit_seconds;
        check_cuda("cudaEventElapsedTime", cudaEventElapsedTime(&timing->device_ms, start, stop));
        timing->operations = issued;
        (void)cudaEventDestroy(start);
        (void)cudaEventDestroy(stop);
        return 0;
    } catch (...) {
        if (start != nullptr) (void)cudaEventDestroy(start);
        if (stop != nullptr) (void)cudaEventDestroy(stop);
        return classify(std::current_exception());
    }
}

}  // extern "C"
