// Host-side admission helpers shared by the C-ABI entry points: checked view
// arithmetic (the rules of detail::validate_checked_view,
// src/device_ops.cpp:114-206, applied to a value snapshot) and the collapsing
// of leading axes into the smallest iteration space the kernels walk.
#pragma once

#include <stdint.h>

#include "common.cuh"

namespace iomb {

struct ViewFacts {
    uint32_t bits;         // leaf width
    uint32_t bytes;        // leaf width in bytes (0 for sub-byte leaves)
    uint32_t leading;      // rank - 2
    uint64_t rows;
    uint64_t cols;
    uint64_t tile_rows;
    uint64_t tile_cols;
    uint64_t plane_bytes;  // tile_rows * tile_cols * tile bytes
    uint64_t planes;       // product of the leading extents
    uint64_t max_plane;    // highest owner plane the view addresses
};

// Validates one view snapshot. Returns IOMB_OK or the status to report.
int check_view(const iomb_view* view, const char* what, ViewFacts* facts);

// True when both snapshots describe the same window of the same owner.
bool same_window(const iomb_view& a, const iomb_view& b);

// True when the byte ranges two views may touch overlap (conservative:
// base + first addressed plane .. base + last addressed plane end).
bool storage_overlaps(const iomb_view& a, const ViewFacts& fa,
                      const iomb_view& b, const ViewFacts& fb);

// Builds the collapsed leading space for `count` operands. `strides[k][axis]`
// are the operands' plane strides aligned to the result's leading axes (zero on
// broadcast axes); they are rewritten in place for the collapsed axes.
void collapse_leading(uint32_t lead_rank, const uint64_t* result_dims,
                      uint64_t strides[][kMaxLead], uint32_t count,
                      Leading* leading);

// Fills the kernel-side operand from a view and its aligned strides.
Operand make_operand(const iomb_view& view, const ViewFacts& facts,
                     const uint64_t* aligned_strides, const Leading& leading,
                     bool bc_rows, bool bc_cols);

// Streaming multiprocessors of the current device (0 when it cannot be read).
int sm_count();

// Raises a kernel's dynamic shared-memory limit to the 227 KiB an SM offers, once per
// kernel and device (the attribute belongs to the function, not to a launch, so it is
// never lowered again: queues on other threads may be launching the same kernel).
int allow_full_shared_memory(const void* kernel);

// One-time set-up of each translation unit's kernels on the current device (behind
// iomb_prepare_device): shared-memory limits, the BF16 SiLU table.
int prepare_rmsnorm_kernels();
int prepare_rmsnorm_long_kernels();
int prepare_silu(cudaStream_t stream);
int prepare_sdpa_kernels();

// Grid size for grid-stride kernels: enough CTAs to fill every SM
// `ctas_per_sm` times, never more than `work_items`.
unsigned grid_for(uint64_t work_items, unsigned ctas_per_sm);

// Grid with one CTA per work item (kernels still loop, so the cap is harmless).
unsigned grid_one_shot(uint64_t work_items);

// cache_append for the leaves of 2, 4 and 6 bits (defined beside the other narrow-leaf movers).
int narrow_append(const iomb_view& source, const ViewFacts& fs, const iomb_view& destination,
                  const ViewFacts& fd, uint64_t a, cudaStream_t stream);

}  // namespace iomb
