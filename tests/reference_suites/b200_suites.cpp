// Runs the reference's own backend-neutral conformance suites
// (test/backend/backend_conformance_*.hpp, included from the reference checkout where it
// lies, never copied) against the B200 backend. The reference's CUDA driver
// (test/cuda/test_cuda_conformance.cpp:163-208) is the pattern: a device triple
// {reference CPU, candidate, foreign} and a storage oracle that seeds and observes whole
// owners with plain cudaMemcpy, independent of the code under test.
//
// TEST INFRASTRUCTURE. Built by `make -C oracle suites` into oracle/_ref/ (it needs the
// reference checkout); tests/test_gpu_reference_suites.py runs the binary on the GPU box.
// Usage: b200_reference_suites [substring of the case names to run]
#include <doctest/doctest.h>

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <memory>
#include <new>
#include <span>
#include <unordered_set>
#include <vector>

#include "backend/backend_conformance_common.hpp"
#include "backend/backend_conformance_copy_storage.hpp"
#include "backend/backend_conformance_embedding.hpp"
#include "backend/backend_conformance_other.hpp"
#include "backend/backend_conformance_rmsnorm.hpp"
#include "backend/backend_conformance_add_gpu.hpp"
#include "backend/backend_conformance_cache_append.hpp"

#include "iom/cpu/device.hpp"
#include "iom_b200_backend.hpp"

namespace {

class HostAllocator final : public iom::Allocator {
public:
    explicit HostAllocator(const iom_conformance::TrafficGate& gate) : gate_(gate) {}

    void* alloc(std::size_t size) override {
        CHECK_MESSAGE(!gate_.armed(), "tensor storage allocated inside an operation");
        void* pointer = ::operator new(size, std::align_val_t(32));
        live_.insert(pointer);
        return pointer;
    }

    void free(void* buffer) override {
        CHECK_MESSAGE(!gate_.armed(), "tensor storage freed inside an operation");
        REQUIRE_MESSAGE(live_.erase(buffer) == 1, "allocator freed an address it never handed out");
        ::operator delete(buffer, std::align_val_t(32));
    }

    void reset() override {}

private:
    const iom_conformance::TrafficGate& gate_;
    std::unordered_set<void*> live_;
};

// The arena of the reference's GPU fixtures (test/cuda/test_cuda_conformance.cpp:85-90).
constexpr std::size_t kArenaBytes = 640u * 1024 * 1024;

struct Devices {
    iom_conformance::TrafficGate gate;
    HostAllocator reference_allocator{gate};
    std::unique_ptr<iom::Device> reference = iom::make_cpu_device(reference_allocator);
    std::unique_ptr<iom::Device> candidate =
            iom::make_b200_device(0, iom::DeviceMemoryConfig{kArenaBytes});
    std::unique_ptr<iom::Device> foreign =
            iom::make_b200_device(0, iom::DeviceMemoryConfig{kArenaBytes});

    [[nodiscard]] iom_conformance::ConformanceDevices conformance() const {
        return {*reference, *candidate, *foreign};
    }
};

class StorageOracle final : public iom_conformance::AcceleratorStorageOracle {
public:
    void seed(iom::TensorView& view, std::span<const std::byte> encoded) override {
        const std::size_t bytes = owner_spec().tiled_storage_nbytes();
        REQUIRE_EQ(encoded.size(), bytes);
        REQUIRE(cudaDeviceSynchronize() == cudaSuccess);
        REQUIRE(cudaMemcpy(view.native_handle(), encoded.data(), bytes, cudaMemcpyHostToDevice)
                == cudaSuccess);
    }

    [[nodiscard]] std::vector<std::byte> observe(const iom::TensorView& view) const override {
        const std::size_t bytes = owner_spec().tiled_storage_nbytes();
        std::vector<std::byte> result(bytes);
        REQUIRE(cudaDeviceSynchronize() == cudaSuccess);
        REQUIRE(cudaMemcpy(result.data(), view.native_handle(), bytes, cudaMemcpyDeviceToHost)
                == cudaSuccess);
        return result;
    }
};

void inject(iom::b200::SubmissionFault fault) {
    iom::b200::inject_submission_fault_for_testing(fault);
}

}  // namespace

TEST_CASE("B200: supported_data_types is the standard 23-entry table") {
    const std::unique_ptr<iom::Device> candidate =
            iom::make_b200_device(0, iom::DeviceMemoryConfig{kArenaBytes});
    iom_conformance::require_standard_capabilities(candidate->supported_data_types());
}

TEST_CASE("B200: storage and host transfers for every leaf type") {
    Devices devices;
    iom_conformance::run_storage_and_transfer_conformance(
            devices.conformance(), devices.candidate->supported_data_types(), &devices.gate);
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: storage oracle identifies a perturbed transfer map") {
    Devices devices;
    const std::span<const iom::DataType> one_type =
            devices.candidate->supported_data_types().subspan(0, 1);
    StorageOracle direct;
    iom_conformance::PermutingStorageOracle perturbed(
            direct, iom_conformance::swap_first_adjacent_slots);
    CHECK_FALSE(iom_conformance::run_storage_oracle_conformance(
            devices.conformance(), one_type, perturbed, &devices.gate, false, false));
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: storage oracle covers every leaf width and padded shape") {
    Devices devices;
    StorageOracle oracle;
    REQUIRE(iom_conformance::run_storage_oracle_conformance(
            devices.conformance(), devices.candidate->supported_data_types(), oracle, &devices.gate));
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: asynchronous copies against the CPU reference") {
    Devices devices;
    StorageOracle oracle;
    iom_conformance::run_async_copy_conformance(
            devices.conformance(), devices.candidate->supported_data_types(), &devices.gate, &oracle);
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: copy validation fails before writes and sequences") {
    Devices devices;
    iom_conformance::run_copy_error_conformance(
            devices.conformance(), devices.candidate->supported_data_types(), &devices.gate);
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: transfer failures keep metadata and ownership") {
    Devices devices;
    iom_conformance::run_transfer_error_conformance(
            devices.conformance(), devices.candidate->supported_data_types(), &devices.gate);
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: deferred queue lifetime and stability") {
    Devices devices;
    iom_conformance::run_lifetime_conformance(
            *devices.candidate, devices.candidate->supported_data_types(), &devices.gate);
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: queue cap and workspace contract") {
    Devices devices;
    iom_conformance::run_memory_contract_conformance(devices.conformance());
}

TEST_CASE("B200: embedding lookup reference, admission, and lifetime") {
    Devices devices;
    StorageOracle oracle;
    // Every payload leaf and every integer id leaf, the {32, 32} status workspace.
    constexpr iom_conformance::EmbeddingDeclaration declaration{
            iom_conformance::kEmbeddingPayloadSpan, iom_conformance::kEmbeddingIdSpan,
            iom_conformance::kEmbeddingPayloadSpan, iom_conformance::kEmbeddingIdSpan,
            iom::WorkspaceRequirements{32, 32}};
    iom_conformance::run_embedding_conformance(
            devices.conformance(), declaration, &devices.gate, &oracle);
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: cache append reference, admission, and lifetime") {
    Devices devices;
    StorageOracle oracle;
    iom_conformance::CacheAppendFaultSeam fault_seam{
            [](iom::DeviceOps&) { inject(iom::b200::SubmissionFault::launch); }};
    iom_conformance::CacheAppendConformanceConfig config{
            devices.conformance(), devices.candidate->supported_data_types(), &oracle, fault_seam,
            {}, nullptr};
    iom_conformance::run_cache_append_conformance(config);
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: RMSNorm reference, admission, and lifetime") {
    Devices devices;
    StorageOracle oracle;
    // The two leaves this backend declares (rmsnorm_supported): BF16 and F32.
    static constexpr iom::DataType leaves[] = {iom::DataType::BF16, iom::DataType::F32};
    iom_conformance::RmsNormConformanceConfig config{
            devices.conformance(), std::span<const iom::DataType>(leaves), &devices.gate, &oracle};
    config.native_failure = iom_conformance::RmsNormNativeFailureSeam{
            [] { inject(iom::b200::SubmissionFault::event_record); },
            [] { inject(iom::b200::SubmissionFault::none); },
            "b200::SubmissionFault::event_record",
            {}};
    iom_conformance::run_rmsnorm_conformance(config);
    CHECK_FALSE(devices.gate.armed());
}

TEST_CASE("B200: binary ADD MUL SUB DIV on the real queue") {
    Devices devices;
    for (const auto operation : {iom_conformance::BinaryOperation::add,
                                 iom_conformance::BinaryOperation::mul,
                                 iom_conformance::BinaryOperation::sub,
                                 iom_conformance::BinaryOperation::div}) {
        iom_conformance::run_gpu_eltwise_conformance(*devices.candidate, operation);
        iom_conformance::run_gpu_eltwise_mapping_conformance(*devices.candidate, operation);
        iom_conformance::run_gpu_exact_alias_conformance(*devices.candidate, operation);
    }
    iom_conformance::run_binary_rank_boundary_conformance(*devices.candidate);
    CHECK_FALSE(devices.gate.armed());
}

int main(int argc, char** argv) {
    return doctest_shim::run_all(argc > 1 ? argv[1] : "") == 0 ? 0 : 1;
}
