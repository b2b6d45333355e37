// Decode attention for callers that must not allocate device memory.
//
// cc_attention_decode_paged needs scratch memory for the partial results of a sequence that is
// split over several CTAs, and its caller has to provide it (cudaMalloc once, or the Gpu object
// does it).  Two kinds of caller of this library cannot do that: a host that has already handed
// every byte of HBM to its KV page pool and weights at start-up, so a later cudaMalloc fails or
// evicts nothing useful; and a model thread that must never block between submissions (the
// contract the reference's `Batch` gives its caller, metal-compute/src/apple.rs:2202-2239),
// for which cudaMalloc and cudaFree are out of the question because both synchronise the whole
// device.  For them the scratch lives in this file, inside the library image: a fixed array in
// device memory that every GPU loading the library holds until the process exits.
#include "../../include/cuda_compute.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "kernels.cuh"

namespace {

// The whole price of this entry point: 16 MiB per GPU, for as long as the library is loaded.
static __device__ __align__(256) unsigned char g_decode_scratch[CC_DECODE_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void *g_scratch_ptr[kMaxDevices] = {};  // device address of the array on each device, once known

}  // namespace

extern "C" size_t cc_decode_static_scratch_bytes(void) { return CC_DECODE_STATIC_SCRATCH_BYTES; }

extern "C" int cc_attention_decode_paged_static(void *stream, const cc_decode_args *args) {
    if (!args) return cc::set_error(CC_DISPATCH, "decode (static scratch): null arguments");
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        cudaGetLastError();
        return cc::set_error(CC_NO_DEVICE, "decode (static scratch): no current CUDA device");
    }
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_scratch_ptr[device]) {
            // In host code `g_decode_scratch` is only a handle for the symbol, not a device
            // address: the address on the current device has to be asked for, once per device.
            void *ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_decode_scratch) != cudaSuccess || !ptr) {
                cudaGetLastError();
                return cc::set_error(CC_COMPILE, "decode (static scratch): the scratch array has no address on this device");
            }
            g_scratch_ptr[device] = ptr;
        }
        scratch = g_scratch_ptr[device];
    }
    const size_t need = cc_decode_workspace_bytes(args->seqs, args->kv_heads, args->max_seq_len, args->window,
                                                  args->pages_per_split);
    if (need > CC_DECODE_STATIC_SCRATCH_BYTES) {
        char text[320];
        snprintf(text, sizeof text,
                 "decode (static scratch): these sizes need %zu bytes of scratch, the built-in array holds %u; "
                 "pass a larger pages_per_split or use cc_attention_decode_paged with your own workspace",
                 need, CC_DECODE_STATIC_SCRATCH_BYTES);
        return cc::set_error(CC_ALLOC, text);
    }
    // The array still holds whatever the previous call left.  The kernel only relies on its
    // arrival counters (one word per sequence and KV head, at the front) starting at zero.
    const size_t counters = (static_cast<size_t>(args->seqs) * args->kv_heads * sizeof(unsigned) + 255) & ~size_t(255);
    if (cudaMemsetAsync(scratch, 0, counters, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        cudaGetLastError();
        return cc::set_error(CC_GPU, "decode (static scratch): could not clear the arrival counters");
    }
    cc_decode_args with_scratch = *args;
    with_scratch.workspace = scratch;
    with_scratch.workspace_bytes = CC_DECODE_STATIC_SCRATCH_BYTES;
    return cc_attention_decode_paged(stream, &with_scratch);
}
