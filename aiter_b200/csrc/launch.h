// Host-side description of one GEMM launch and the configuration record the dispatcher works with.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include <sstream>
#include <string>

namespace b200 {

// Throwing check used below the C ABI; the ABI wrapper turns it into "-1 + thread-local message"
// (the reference's AITER_CHECK + aiter_safe_call pair, csrc/include/aiter_hip_common.h:67-74).
template <typename... Args>
[[noreturn]] inline void fail(Args&&... args)
{
    std::ostringstream os;
    (os << ... << args);
    throw std::runtime_error(os.str());
}
#define B200_CHECK(cond, ...)            \
    do                                   \
    {                                    \
        if(!(cond))                      \
            ::b200::fail(__VA_ARGS__);   \
    } while(0)
#define B200_CUDA(expr)                                                                     \
    do                                                                                      \
    {                                                                                       \
        cudaError_t e_ = (expr);                                                            \
        if(e_ != cudaSuccess)                                                               \
            ::b200::fail(#expr, " failed: ", cudaGetErrorString(e_));                       \
    } while(0)

enum ProblemKind : int
{
    PK_BF16   = 0, // bf16 x bf16
    PK_MXFP8  = 1, // e4m3 x e4m3, e8m0 per 32
    PK_MXFP4  = 2, // e2m1 x e2m1, e8m0 per 32
    PK_MXF8F4 = 3, // e4m3 activations x e2m1 weights
    PK_NVFP4  = 4, // e2m1 x e2m1, e4m3 per 16 (the per-tensor scales ride in alpha)
};

struct Operand
{
    const void* ptr = nullptr;
    long long rows  = 0;
    long long kbytes = 0;    // bytes along K per row
    long long ld_bytes = 0;  // row pitch in bytes (row-major mode only)
    int mode = 0;            // OperandMode
    long long batch_stride_bytes = 0; // batched problems (mode OPM_BATCHED): bytes between two matrices
    long long batch = 1;              //                                       number of matrices
};

struct ScaleOperand
{
    const void* ptr = nullptr;
    int wire = 0;              // SfWire
    long long padded_rows = 0; // rows of the (padded) scale array, multiple of 32
    long long padded_cols = 0; // scale columns of the (padded) array
};

struct KernelConfig
{
    int swap   = -1; // 1: weights fill the 128-row slot; 0: activations do; -1: choose
    int bn     = 0;  // UMMA N (0: choose)
    int stages = 0;  // 0: choose
    int log2_splitk = -1; // -1: choose
    int cg = 0;      // CTAs per tile: 1, or 2 (a 256-row tile on a CTA pair); 0: choose
    int decode_stages = 0; // set by the heuristic only: the decode kernel runs with this many stages, a CTA alone on its SM
                           // (0: as many as keep two CTAs on an SM, or what `stages` names)
};

// Caller-provided scratch for a launch that must not allocate: split-K partials, ticket counters and the
// status record all live in memory the caller already owns.
struct ExternalScratch
{
    float* partial          = nullptr;
    size_t partial_bytes    = 0;
    unsigned int* counter   = nullptr; // zero before the launch
    int counter_slots       = 0;
    unsigned int* status    = nullptr; // 4 words
};

struct GemmProblem
{
    int kind = PK_BF16;
    long long M = 0, N = 0, K = 0; // K in elements
    Operand act, wgt;
    ScaleOperand act_sf, wgt_sf;
    void* out = nullptr;
    long long ldo = 0;          // row pitch in output elements (bytes for the e2m1 / e4m3 outputs)
    int out_mode = 0;           // OutMode: bf16, fp16, fp32, packed e2m1 (no scale), e4m3 + UE8M0 per 128 columns
    void* out_scale = nullptr;  // OUT_MXFP8: [M, N/128] bytes, filled in the packed (M/64, N/128, 16, 4) order
    int noscale = 0;            // ignore the block scales (the reference's fp4-output GEMM is its "noscale" kernel)
    long long batch = 1;        // [batch, M, K] x [batch, N, K] -> [batch, M, N] in one launch (bf16 operands, row-major)
    long long out_batch_stride = 0;  // output elements between two matrices
    long long bias_batch_stride = 0; // bias elements between two matrices' bias vectors (0: shared)
    const void* bias = nullptr; // indexed by n
    int bias_is_bf16 = 0;
    float alpha = 1.f, beta = 1.f;
    int device = 0;
    cudaStream_t stream = nullptr;
    KernelConfig cfg;
    const ExternalScratch* scratch = nullptr; // null: the library's own per-device / per-stream buffers
};

// Fills the unset fields of cfg with the heuristic choice for (kind, M, N, K).
void choose_config(int kind, long long M, long long N, long long K, int num_sms, KernelConfig& cfg);
// "tc5_<128|256>x<bn>_<n|t>_s<stages>" <-> KernelConfig (t = swapped / transposed store; 256 = CTA pair).
std::string config_name(const KernelConfig& cfg);
bool parse_config_name(const char* name, KernelConfig& cfg);
// kernelId <-> configuration (index into the fixed menu printed by aiter_b200_kernel_list()).
bool config_from_id(int kernel_id, KernelConfig& cfg);
const char* kernel_menu_text();

void launch_gemm(const GemmProblem& prob);

// FP8 x FP8 with fp32 scales per 128-wide K block (x_scale[m][kb] at x_scale + m*xs_stride_m + kb*xs_stride_k,
// w_scale [ceil(N/128)][K/128] dense), bf16 output.
struct BlockScaleProblem
{
    long long M = 0, N = 0, K = 0;
    Operand act, wgt;
    const float* x_scale = nullptr;
    long long xs_stride_m = 0, xs_stride_k = 0;
    const float* w_scale = nullptr;
    // both scale tensors hold UE8M0 bytes instead of floats (same shapes and strides, in bytes): powers of two ride
    // the block-scaled MMA, so the problem runs on the MXFP8 kernel after a small expansion of the scales (up to 64
    // rows without a caller-chosen configuration: on the few-rows kernel, which reads the bytes itself)
    bool scales_are_e8m0 = false;
    KernelConfig cfg;             // e8m0 path only: a caller-chosen MXFP8 kernel configuration (unset fields: heuristic)
    bool cfg_given = false;
    void* out = nullptr;
    long long ldo = 0;
    int out_mode = 0;             // OutMode: bf16, fp16 or fp32
    // fp32-scale kernels: which one runs and its K split, for tuned tables (0 / -1: the launcher's own cost model).
    // Names: "bs_fewrows" (<= 64 rows), "bs_128x128", "bs_256x256" (CTA pairs), each with an optional "_k<log2 split>".
    int variant = 0;              // 1 few-rows, 2 128x128 single CTA, 3 256x256 CTA pair
    int log2_splitk = -1;
    int device = 0;
    cudaStream_t stream = nullptr;
};
void launch_blockscale(const BlockScaleProblem& prob);
// "bs_fewrows" | "bs_128x128" | "bs_256x256" [+ "_k<n>"] -> (variant, log2 split); false when the name is not one of these
bool parse_blockscale_name(const char* name, int& variant, int& log2_splitk);
void read_device_status(int device, unsigned int out_words[4]);
// Bound of every in-kernel wait on `device` (1 ms .. 10 s, default 1 s) and the test hook that makes the persistent
// kernel's scale producer issue nothing, so that a wait runs out.  Synchronises the device.
void set_wait_control(int device, unsigned long long limit_ns, int withhold_scales);
unsigned long long launch_count();
void count_launch(); // kernels launched outside launch.cu report themselves here
int device_sm_count(int device);

} // namespace b200
