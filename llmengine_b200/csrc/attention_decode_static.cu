// llme_attention_decode_static: the split-context decode attention of attention_fast.cu with its
// scratch memory kept in a device array of this library, for callers that cannot allocate.
// What it is for, its limits and its rules are in attention_decode_static.h.  It has no
// counterpart in the reference project.
//
// The kernels are the ones of attention_fast.cu, compiled into this library unchanged; this file
// only adds the array, the per-device look-up of its address and the entry point.
#include "attention_fast.cu"
#include "attention_decode_static.h"

static_assert(sizeof(LlmeDecodeArgs) == sizeof(FastAttnArgs), "the public argument block must match the kernels'");

// The partial results of the context splits.  Device code could name this array directly; host
// code must not pass its name to a kernel (on the host the name is only a stand-in, not a device
// address), so the address is asked for below, once per device.
static __device__ __align__(256) float llme_static_scratch[LLME_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES] = {nullptr};
}  // namespace

LLME_API long long llme_attention_decode_static_capacity(void) { return LLME_STATIC_SCRATCH_FLOATS; }

LLME_API int llme_attention_decode_static(const LlmeDecodeArgs* public_args, cudaStream_t stream) {
    if (!public_args) LLME_REFUSE("attention_decode_static: null argument block");
    FastAttnArgs a = *reinterpret_cast<const FastAttnArgs*>(public_args);
    if (a.n_rows <= 0) return 0;
    if (a.nh <= 0 || a.splits < 1) LLME_REFUSE("attention_decode_static: %d heads, %d splits: both must be positive", a.nh, a.splits);
    const long long need = llme_attention_decode_scratch_floats(a.n_rows, a.nh, a.splits);
    if (need > (long long)LLME_STATIC_SCRATCH_FLOATS)
        LLME_REFUSE("attention_decode_static: %d requests x %d heads x %d splits need %lld scratch values, "
                    "the built-in array holds %d; use fewer splits or llme_attention_decode with your own buffer",
                    a.n_rows, a.nh, a.splits, need, (int)LLME_STATIC_SCRATCH_FLOATS);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) LLME_REFUSE("attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (device < 0 || device >= MAX_DEVICES) LLME_REFUSE("attention_decode_static: device index %d is not supported", device);
    if (!g_scratch_address[device]) {
        // First call on this device (it is the current one): look up where the array lives there.
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, llme_static_scratch);
        if (e != cudaSuccess || !p)
            LLME_REFUSE("attention_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_scratch_address[device] = p;
    }
    a.scratch = g_scratch_address[device];
    return llme_attention_decode(&a, stream);
}
