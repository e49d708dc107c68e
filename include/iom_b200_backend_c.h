/*
 * C driver interface of the C++ B200 backend (libiom_b200_backend.so).
 *
 * The backend itself is C++ (include/iom_b200_backend.hpp: make_b200_device returns an
 * iom::Device for IOM's own facade). This header lets a program without a C++ toolchain
 * of the reference's (a benchmark, a script) create that device and run sequences of
 * facade operations on it with device-side timing. It has no counterpart in the
 * reference: every call below is a thin wrapper over the reference's public interface
 * (include/iom/device.hpp:57-131, include/iom/tensor.hpp:322-342, include/iom/iom.hpp:105-373)
 * on a device from make_b200_device.
 *
 * Handles are opaque pointers; a null handle or a nonzero status means failure and
 * iomb_backend_last_error() describes it. Destroy views before their tensor, tensors,
 * workspaces and queues before their device.
 */
#ifndef IOM_B200_BACKEND_C_H
#define IOM_B200_BACKEND_C_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* iomb_backend_last_error(void);

/* make_b200_device(ordinal, {arena_bytes}, {max_in_flight}); max_in_flight 0 = the default. */
void* iomb_backend_device_create(uint32_t ordinal, uint64_t arena_bytes, uint32_t max_in_flight);
void iomb_backend_device_destroy(void* device);

/* Device::create_ops / create_tensor / create_workspace. */
void* iomb_backend_queue_create(void* device);
void iomb_backend_queue_destroy(void* queue);
void* iomb_backend_tensor_create(void* device, const uint64_t* dims, uint32_t rank, uint32_t dtype);
void iomb_backend_tensor_destroy(void* tensor);
/* Owner storage (device address) and its size: for filling inputs without a host pass. */
void* iomb_backend_tensor_address(void* tensor);
uint64_t iomb_backend_tensor_nbytes(void* tensor);
void* iomb_backend_workspace_create(void* device, uint64_t bytes);
void iomb_backend_workspace_destroy(void* workspace);
void* iomb_backend_workspace_address(void* workspace);

/* Tensor::view and the view transforms (include/iom/tensor.hpp:322-329). */
void* iomb_backend_view_full(void* tensor);
void* iomb_backend_view_select(void* view, uint64_t dim, uint64_t index);
void* iomb_backend_view_slice(void* view, uint64_t dim, uint64_t first, uint64_t count, uint64_t step);
void iomb_backend_view_destroy(void* view);

/* One operation of a program. Unused fields are zero. */
typedef enum iomb_backend_opcode {
    IOMB_BACKEND_ADD = 0,           /* views: lhs, rhs, out */
    IOMB_BACKEND_MUL = 1,
    IOMB_BACKEND_SUB = 2,
    IOMB_BACKEND_DIV = 3,
    IOMB_BACKEND_RMSNORM = 4,       /* views: x, scale, out; eps */
    IOMB_BACKEND_ADD_RMSNORM = 5,   /* views: x, residual, scale, sum, out; eps */
    IOMB_BACKEND_COPY = 6,          /* views: source, destination */
    IOMB_BACKEND_EMBEDDING = 7,     /* views: table, indices, out; workspace (>= 32 bytes) */
    IOMB_BACKEND_CACHE_APPEND = 8,  /* views: source, destination; a */
    IOMB_BACKEND_CACHE_APPEND_BATCHED = 9, /* views: source, destination; workspace = control */
    IOMB_BACKEND_SILU = 10,         /* views: x, y */
    IOMB_BACKEND_SILU_MUL = 11,     /* views: x, up, out */
    IOMB_BACKEND_ROPE = 12,         /* views: x, out; a; theta */
    IOMB_BACKEND_CAST = 13,         /* views: source, destination */
    IOMB_BACKEND_SUMSQ = 14,        /* views: x; workspace */
    IOMB_BACKEND_FROM_HOST = 15,    /* views: destination; host, host_bytes; workspace = staging */
    IOMB_BACKEND_TO_HOST = 16,      /* views: source; host, host_bytes; workspace = staging */
    IOMB_BACKEND_WAIT = 17          /* waits for every token issued so far in this pass */
} iomb_backend_opcode;

typedef struct iomb_backend_op {
    uint32_t opcode;
    uint32_t reserved;
    void* views[5];
    void* workspace;
    void* host;
    uint64_t host_bytes;
    uint64_t a;
    double theta;
    float eps;
    float reserved2;
} iomb_backend_op;

typedef struct iomb_backend_timing {
    double host_seconds;     /* steady clock around all passes, submission to last wait */
    double submit_seconds;   /* of which: time spent inside the submitting calls */
    float device_ms;         /* CUDA events on the queue's stream around all passes */
    uint32_t reserved;
    uint64_t operations;     /* facade operations issued (passes x operations per pass) */
} iomb_backend_timing;

/* Run modes. */
#define IOMB_BACKEND_EAGER 0u        /* every pass issues the operations one by one */
#define IOMB_BACKEND_WAIT_EACH 1u    /* as EAGER, waiting for each token before the next call */
#define IOMB_BACKEND_RECORDED 2u     /* the pass is recorded once (b200::capture_begin/_end) and
                                        replayed: one submission per pass */

/*
 * Runs the program `passes` times on `queue` after `warmup` untimed passes. Host transfer
 * operations are the contract's synchronous calls. Returns 0, or the failure class of
 * the first failing call (1 invalid argument, 2 out of range, 3 overflow, 4 resource
 * exhausted, 5 other, 6 unknown); a negative oid from a facade call is reported as 5 with
 * the oid in the error text.
 */
int iomb_backend_run(void* queue, const iomb_backend_op* operations, uint32_t count,
                     uint32_t warmup, uint32_t passes, uint32_t mode,
                     iomb_backend_timing* timing);

#ifdef __cplusplus
}
#endif

#endif
