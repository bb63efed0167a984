// An MXFP8 GEMM entry point for callers that cannot allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits - a serving loop that has handed all of its
// memory to one arena up front and treats any later driver allocation as a bug, a plugin loaded into a host
// process whose allocator it must not touch, or a latency-critical path where an allocation (which can
// synchronise the device) is unacceptable.  The regular entry points keep their split-K partial sums,
// their per-tile ticket counters and their status record in buffers they cudaMalloc on first use and grow
// on demand; this one keeps all three in one fixed array that is part of the library image.
//
// The price: the array (8 MiB + 32 KiB) is resident on every GPU that loads the library until the process
// exits, shapes whose split-K partials do not fit are refused, and all calls share the one array - it keeps
// the previous call's contents, and two calls that overlap on the GPU (different streams, or the same GEMM
// launched again before the first finished on another stream) race on it.
#include "../../include/aiter_b200.h"
#include "abi_checks.h"
#include "gemm_common.cuh"
#include "launch.h"

#include <mutex>
#include <string>

using namespace b200;

namespace {

constexpr size_t kStatusBytes    = 256;                 // 4 words used
constexpr int kCounterSlotsFixed = 4096;                // ticket counters, one per output tile
constexpr size_t kCounterBytes   = 32 * 1024 - kStatusBytes;
constexpr size_t kPartialBytes   = 8u << 20;            // fp32 split-K partial sums
constexpr size_t kScratchBytes   = kStatusBytes + kCounterBytes + kPartialBytes;
static_assert(kCounterSlotsFixed * sizeof(unsigned int) <= kCounterBytes, "counter region too small");

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress - it is NOT a
// device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct PerDevice
{
    bool ready = false;
    unsigned char* base = nullptr; // device address of g_noalloc_scratch on that device
};
std::mutex g_setup_mutex;
PerDevice g_per_device[64];

// First call on a device: look up where the array lives on that device.  Nothing is allocated, but this is
// a runtime call that should not happen while a stream is being captured - make the first call beforehand.
unsigned char* scratch_base(int device)
{
    B200_CHECK(device >= 0 && device < 64, "device index out of range");
    std::lock_guard<std::mutex> lk(g_setup_mutex);
    PerDevice& pd = g_per_device[device];
    if(!pd.ready)
    {
        int prev = 0;
        B200_CUDA(cudaGetDevice(&prev));
        B200_CUDA(cudaSetDevice(device));
        void* ptr     = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        cudaSetDevice(prev);
        if(e != cudaSuccess || ptr == nullptr)
            fail("cudaGetSymbolAddress(static scratch) failed on device ", device, ": ", cudaGetErrorString(e));
        pd.base  = static_cast<unsigned char*>(ptr);
        pd.ready = true;
    }
    return pd.base;
}

} // namespace

// defined in abi.cu: stores the message where aiter_get_last_error() finds it
void aiter_b200_set_last_error(const std::string& msg);

extern "C" int aiter_b200_gemm_a8w8_mxfp8_noalloc(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA,
                                                  aiter_tensor_t* ScaleB, aiter_tensor_t* out, int a_preshuffle,
                                                  int log2_k_split, void* stream)
{
    try
    {
        const char* fn = "aiter_b200_gemm_a8w8_mxfp8_noalloc";
        // the same checks as the regular MXFP8 entry point: nothing else stands between a wrong argument and a
        // kernel reading the wrong memory
        require_tensor(A, fn, "A", 2);
        require_tensor(B, fn, "B", 2);
        require_tensor(out, fn, "out", 2);
        B200_CHECK(is_byte_dtype(A->dtype_) && is_byte_dtype(B->dtype_), fn, ": A and B must be 1-byte (fp8) tensors (got ",
                   dtype_name(A->dtype_), ", ", dtype_name(B->dtype_), ")");
        B200_CHECK(out->dtype_ == AITER_DTYPE_bf16, fn, " only supports BFloat16 output");
        B200_CHECK(a_preshuffle == 0 || a_preshuffle == 1, fn, " a_preshuffle must be 0 or 1");
        B200_CHECK(log2_k_split >= -1 && log2_k_split <= 8, fn, ": log2 of the K split must be between 0 and 8 (got ", log2_k_split, ")");
        const long long M = A->shape[0], N = B->shape[0], K = A->shape[1];
        B200_CHECK(K % 128 == 0, fn, " K must be divisible by 128 (got K=", K, ")");
        B200_CHECK(B->shape[1] == K, fn, ": B must be [N, K]");
        B200_CHECK(out->shape[0] >= M && out->shape[1] == N, fn, ": out must be [>=M, N]");
        require_rows_contiguous(out, fn, "out");
        require_dense(A, fn, "A");
        require_dense(B, fn, "B");
        const ScaleOperand sfa = scale_operand(ScaleA, SFW_G1250, fn, "ScaleA");
        const ScaleOperand sfb = scale_operand(ScaleB, SFW_G1250, fn, "ScaleB");
        require_same_device(A, B, fn, "B");
        require_same_device(A, ScaleA, fn, "ScaleA");
        require_same_device(A, ScaleB, fn, "ScaleB");
        require_same_device(A, out, fn, "out");

        unsigned char* base = scratch_base(A->device_id);
        ExternalScratch sc;
        sc.status        = reinterpret_cast<unsigned int*>(base);
        sc.counter       = reinterpret_cast<unsigned int*>(base + kStatusBytes);
        sc.counter_slots = kCounterSlotsFixed;
        sc.partial       = reinterpret_cast<float*>(base + kStatusBytes + kCounterBytes);
        sc.partial_bytes = kPartialBytes;

        int prev = 0;
        B200_CUDA(cudaGetDevice(&prev));
        if(prev != A->device_id)
            B200_CUDA(cudaSetDevice(A->device_id));
        // the array keeps the last call's contents: the tickets must start at zero (partials are fully overwritten
        // before they are read).  The status record is NOT cleared here: a failure stays on record until
        // aiter_b200_noalloc_status fetches it.
        cudaError_t e = cudaMemsetAsync(base + kStatusBytes, 0, kCounterBytes, static_cast<cudaStream_t>(stream));
        if(prev != A->device_id)
            cudaSetDevice(prev);
        B200_CUDA(e);

        GemmProblem p;
        p.kind = PK_MXFP8;
        p.M = M; p.N = N; p.K = K;
        p.act    = Operand{A->ptr, M, K, K, a_preshuffle ? OPM_A2X128 : OPM_ROWMAJOR};
        p.wgt    = Operand{B->ptr, N, K, K, OPM_TILE16};
        p.act_sf = sfa;
        p.wgt_sf = sfb;
        p.out    = out->ptr;
        p.ldo    = out->strides[0];
        p.device = A->device_id;
        p.stream = static_cast<cudaStream_t>(stream);
        p.cfg.log2_splitk = log2_k_split;
        p.scratch = &sc;
        launch_gemm(p);
        aiter_b200_set_last_error("");
        return 0;
    }
    catch(const std::exception& ex)
    {
        aiter_b200_set_last_error(ex.what());
    }
    catch(...)
    {
        aiter_b200_set_last_error("unknown C++ exception");
    }
    return -1;
}

// The status record of the allocation-free entry point (four words at the start of the static array: code, CTA,
// K slice, iteration; all zero = no wait ever ran out).  Synchronises the device, copies the record out and clears
// it.  Allocates nothing: the copy goes through the address cudaGetSymbolAddress returned at set-up.
extern "C" int aiter_b200_noalloc_status(int device, unsigned int out_words[4])
{
    try
    {
        B200_CHECK(out_words != nullptr, "aiter_b200_noalloc_status: out_words is required");
        unsigned char* base = scratch_base(device);
        int prev = 0;
        B200_CUDA(cudaGetDevice(&prev));
        if(prev != device)
            B200_CUDA(cudaSetDevice(device));
        cudaError_t e = cudaDeviceSynchronize();
        if(e == cudaSuccess)
            e = cudaMemcpy(out_words, base, 4 * sizeof(unsigned int), cudaMemcpyDeviceToHost);
        if(e == cudaSuccess)
            e = cudaMemset(base, 0, kStatusBytes);
        if(prev != device)
            cudaSetDevice(prev);
        B200_CUDA(e);
        aiter_b200_set_last_error("");
        return 0;
    }
    catch(const std::exception& ex)
    {
        aiter_b200_set_last_error(ex.what());
    }
    catch(...)
    {
        aiter_b200_set_last_error("unknown C++ exception");
    }
    return -1;
}
