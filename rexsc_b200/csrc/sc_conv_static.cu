// SC conv2d forward for callers that must not allocate device memory.
//
// Some hosts of this library cannot hand it a workspace: a plugin loaded into an application whose own pool
// already owns the device memory (a cudaMalloc from the plugin fails or steals from that pool), or a serving
// loop that forbids allocation calls after start-up because cudaMalloc and cudaFree synchronise the device.
// For them this file keeps the scratch of the SC conv forward in a fixed array that is part of the library
// image, and the entry point below runs the ordinary forward on it: it calls no cudaMalloc, no cudaFree and
// no allocating library routine.
//
// What that costs and what the caller has to know:
//   * every GPU on which the library is loaded holds REXSC_STATIC_SCRATCH_BYTES (32 MiB) until the process
//     exits, whether or not this entry point is ever called;
//   * a call whose scratch need (rexsc_sc_conv2d_workspace_size) exceeds that size is rejected with
//     REXSC_E_STATIC_SCRATCH and nothing is launched;
//   * every call asks the runtime for the array's address on the current device (cudaGetSymbolAddress: no
//     allocation, valid again after a device reset).  The FIRST call on a device may load the library's module
//     there; make that first call during set-up, before any stream capture begins;
//   * all calls share the one array and it keeps whatever the previous call left in it.  Each call rewrites
//     every region it later reads (stream tables, activation words, weight words, sign words) and clears the
//     status word first, so stale contents never reach a result -- but two calls that overlap on the GPU
//     (different streams, or different host threads without ordering) race on it.  Serialise them.
#include "common.cuh"

#define REXSC_STATIC_SCRATCH_BYTES (32u << 20)

// The scratch itself.  In host code this name is only a handle for the runtime's symbol table, not a device
// address: it must never be passed to a kernel.  The address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[REXSC_STATIC_SCRATCH_BYTES];

namespace {

// Device address of the static scratch on the CURRENT device.  Asked of the runtime on every call instead of being
// cached: the lookup allocates nothing and costs about a microsecond once the module is loaded, and an address kept
// across a cudaDeviceReset (or any other re-creation of the context) would be stale.
int static_scratch_address(void **out)
{
    void *ptr = nullptr;
    REXSC_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) return REXSC_E_CUDA;
    *out = ptr;
    return REXSC_OK;
}

} // namespace

extern "C" size_t rexsc_sc_conv2d_static_scratch_bytes(void) { return REXSC_STATIC_SCRATCH_BYTES; }

extern "C" int rexsc_sc_conv2d_fwd_static(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight,
                                          int16_t *d_out_pos, int16_t *d_out_neg, void *stream)
{
    const size_t need = rexsc_sc_conv2d_workspace_size(desc);
    if (need == 0) {
        // let the ordinary path name the reason (bad argument, unsupported configuration, too long)
        rexsc::ConvPlan p;
        const int rc = rexsc::make_conv_plan(desc, &p);
        return rc != REXSC_OK ? rc : REXSC_E_BAD_ARG;
    }
    if (need > REXSC_STATIC_SCRATCH_BYTES) return REXSC_E_STATIC_SCRATCH;
    void *scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != REXSC_OK) return rc;
    return rexsc::conv_forward(desc, d_act, d_weight, d_out_pos, d_out_neg, scratch, REXSC_STATIC_SCRATCH_BYTES,
                               (cudaStream_t)stream);
}

// Device status of the calls made through rexsc_sc_conv2d_fwd_static on the current device: synchronises `stream`
// and reads the status word at the head of the built-in scratch, exactly as rexsc_workspace_status does for a
// caller-owned workspace.  Allocates nothing.
extern "C" int rexsc_sc_conv2d_static_status(void *stream)
{
    void *scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != REXSC_OK) return rc;
    return rexsc_workspace_status(scratch, stream);
}
