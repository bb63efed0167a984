// extern "C" entry points: argument checking, aiter_tensor_t -> GemmProblem, error bridge.
#include "../../include/aiter_b200.h"
#include "abi_checks.h"
#include "gemm_common.cuh"
#include "launch.h"
#include "quant_mx.cuh"

#include <climits>
#include <string>

using namespace b200;

static thread_local std::string g_last_error;
static thread_local std::string g_heuristic_name;

// used by entry points that live in other translation units
void aiter_b200_set_last_error(const std::string& msg) { g_last_error = msg; }

template <typename Fn>
static int safe_call(Fn&& fn)
{
    g_last_error.clear();
    try
    {
        fn();
        return 0;
    }
    catch(const std::exception& e)
    {
        g_last_error = e.what();
    }
    catch(...)
    {
        g_last_error = "unknown C++ exception";
    }
    return -1;
}

// OutMode of a plain (not re-quantised) output tensor, or -1
static int plain_out_mode(int dtype)
{
    return dtype == AITER_DTYPE_bf16 ? OUT_BF16 : dtype == AITER_DTYPE_fp16 ? OUT_F16 : dtype == AITER_DTYPE_fp32 ? OUT_F32 : -1;
}

static void set_out(GemmProblem& p, const aiter_tensor_t* out, const char* fn, long long M, long long N)
{
    require_tensor(out, fn, "out", 2);
    B200_CHECK(out->dtype_ == AITER_DTYPE_bf16, fn, " only support BFloat16 output now!");
    B200_CHECK(out->shape[0] >= M && out->shape[1] == N, fn, ": out must be [>=", M, ", ", N, "] (got [", out->shape[0],
               ", ", out->shape[1], "])");
    require_rows_contiguous(out, fn, "out");
    p.out = out->ptr;
    p.ldo = out->strides[0];
}

static void apply_config(GemmProblem& p, const char* kernelName, int log2_splitk, const char* fn)
{
    // -1 (Python None) leaves the split to the heuristic; anything else is log2 of the number of K slices
    B200_CHECK(log2_splitk >= -1 && log2_splitk <= 8, fn, ": log2 of the K split must be between 0 and 8 (got ", log2_splitk, ")");
    p.cfg.log2_splitk = log2_splitk;
    if(kernelName != nullptr && kernelName[0] != 0) // a "_k<n>" suffix of the name overrides the split argument
        B200_CHECK(parse_config_name(kernelName, p.cfg), fn, ": not find kernel ", kernelName);
}

// ------------------------------------------------------------------------------------------- MXFP4
static void run_mxfp4(const char* fn, aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* A_scale,
                      aiter_tensor_t* B_scale, aiter_tensor_t* out, aiter_tensor_t* bias, float alpha, float beta,
                      int a_mode, int b_mode, int wire, const KernelConfig& cfg, void* stream)
{
    require_tensor(A, fn, "A", 2);
    require_tensor(B, fn, "B", 2);
    B200_CHECK(A->dtype_ == AITER_DTYPE_fp4x2 || A->dtype_ == AITER_DTYPE_u8, fn, " Unsupported input_type:",
               dtype_name(A->dtype_));
    B200_CHECK(B->dtype_ == AITER_DTYPE_fp4x2 || B->dtype_ == AITER_DTYPE_u8, fn, " Unsupported input_type:",
               dtype_name(B->dtype_));
    const long long M = A->shape[0], N = B->shape[0], Kb = A->shape[1];
    B200_CHECK(B->shape[1] == Kb, fn, ": A and B disagree on K (", Kb * 2, " vs ", B->shape[1] * 2, ")");
    B200_CHECK(Kb % 16 == 0, fn, ": K must be a multiple of 32");
    require_rows_contiguous(A, fn, "A");
    require_dense(B, fn, "B");
    GemmProblem p;
    p.kind = PK_MXFP4;
    p.M = M; p.N = N; p.K = Kb * 2;
    p.act = Operand{A->ptr, M, Kb, A->strides[0], a_mode};
    if(a_mode != OPM_ROWMAJOR)
        require_dense(A, fn, "A");
    p.wgt    = Operand{B->ptr, N, Kb, Kb, b_mode};
    p.act_sf = scale_operand(A_scale, wire, fn, "A_scale");
    p.wgt_sf = scale_operand(B_scale, wire, fn, "B_scale");
    set_out(p, out, fn, M, N);
    if(bias != nullptr)
    {
        B200_CHECK(bias->dtype_ == AITER_DTYPE_fp32 && static_cast<long long>(bias->numel_) == N, fn,
                   ": bias must be fp32 with N elements");
        p.bias = bias->ptr;
    }
    p.alpha  = alpha;
    p.beta   = beta;
    p.device = A->device_id;
    p.stream = static_cast<cudaStream_t>(stream);
    p.cfg    = cfg;
    launch_gemm(p);
}

extern "C" int gemm_a4w4_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* A_scale, aiter_tensor_t* B_scale,
                             aiter_tensor_t* out, const char* kernelName, aiter_tensor_t* bias, float alpha, float beta,
                             int bpreshuffle, int log2_k_split, void* stream)
{
    return safe_call([&] {
        GemmProblem tmp;
        apply_config(tmp, kernelName, log2_k_split, "gemm_a4w4_asm");
        run_mxfp4("gemm_a4w4_asm", A, B, A_scale, B_scale, out, bias, alpha, beta, OPM_ROWMAJOR,
                  bpreshuffle ? OPM_TILE16 : OPM_ROWMAJOR, SFW_E8M0_SHUFFLE, tmp.cfg, stream);
    });
}

extern "C" int gemm_a4w4_blockscale(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                    aiter_tensor_t* w_scale, aiter_tensor_t* Out, int splitK, const char* kernelName,
                                    void* stream)
{
    return safe_call([&] {
        GemmProblem tmp;
        apply_config(tmp, kernelName, splitK, "gemm_a4w4_blockscale");
        run_mxfp4("gemm_a4w4_blockscale", XQ, WQ, x_scale, w_scale, Out, nullptr, 1.f, 0.f, OPM_ROWMAJOR, OPM_TILE16,
                  SFW_E8M0_SHUFFLE, tmp.cfg, stream);
    });
}

extern "C" int gemm_a4w4_blockscale_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                         aiter_tensor_t* w_scale, aiter_tensor_t* Out, int kernelId, int splitK,
                                         void* stream)
{
    return safe_call([&] {
        KernelConfig cfg;
        B200_CHECK(config_from_id(kernelId, cfg), "gemm_a4w4_blockscale_tune: Kernel id ", kernelId, " not found");
        cfg.log2_splitk = splitK;
        run_mxfp4("gemm_a4w4_blockscale_tune", XQ, WQ, x_scale, w_scale, Out, nullptr, 1.f, 0.f, OPM_ROWMAJOR, OPM_TILE16,
                  SFW_E8M0_SHUFFLE, cfg, stream);
    });
}

// The F4GEMM family (aiter/ops/gemm_op_a4w4.py:290-443): packed e2m1 operands in 16x16-byte tiles (A optionally row-major),
// scales in tiles of 32 rows x 4 e8m0 bytes (MXFP4, one per 32 elements) or 32 rows x 8 e4m3 bytes (NVFP4, one per 16
// elements, `nv`), and for NVFP4 the product of the two per-tensor scales folded into the result.
static void run_f4gemm(const char* fn, bool nv, float global_scale, aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA,
                       aiter_tensor_t* ScaleB, aiter_tensor_t* out, aiter_tensor_t* out_scale, const char* kernelName,
                       int a_preshuffle, void* stream)
{
    {
        B200_CHECK(a_preshuffle == 0 || a_preshuffle == 1, fn, " a_preshuffle must be 0 or 1");
        GemmProblem tmp;
        apply_config(tmp, kernelName, -1, fn);
        B200_CHECK(A != nullptr && A->ndim == 2 && (A->shape[1] * 2) % 256 == 0, fn, " K must be divisible by 256");
        require_tensor(out, fn, "out", 2);
        const bool out_fp4 = (out->dtype_ == AITER_DTYPE_fp4x2 || out->dtype_ == AITER_DTYPE_u8);
        const bool out_fp8 = (out->dtype_ == AITER_DTYPE_fp8);
        if(!out_fp4 && !out_fp8 && !nv)
        {
            B200_CHECK(out_scale == nullptr, fn, ": out_scale goes with the fp8 output only");
            run_mxfp4(fn, A, B, ScaleA, ScaleB, out, nullptr, 1.f, 0.f, a_preshuffle ? OPM_TILE16 : OPM_ROWMAJOR, OPM_TILE16, SFW_G1250,
                      tmp.cfg, stream);
            return;
        }
        // Low-precision outputs (the reference's gemm_a4w4o4 / gemm_a4w4o8, aiter/ops/gemm_op_a4w4.py:457-567):
        //   fp4x2 / uint8 [M, N/2]: packed e2m1 of the product WITHOUT the block scales (its fp4-output kernel ignores them;
        //   the per-tensor scales of NVFP4 still apply);
        //   fp8 [M, N] + out_scale [M, N/128] e8m0 in the packed (M/64, N/128, 16, 4) byte order.
        require_tensor(A, fn, "A", 2);
        require_tensor(B, fn, "B", 2);
        const long long M = A->shape[0], N = B->shape[0], Kb = A->shape[1];
        B200_CHECK(B->shape[1] == Kb, fn, ": A and B disagree on K");
        B200_CHECK(A->dtype_ == AITER_DTYPE_fp4x2 || A->dtype_ == AITER_DTYPE_u8, fn, " Unsupported input_type:", dtype_name(A->dtype_));
        B200_CHECK(B->dtype_ == AITER_DTYPE_fp4x2 || B->dtype_ == AITER_DTYPE_u8, fn, " Unsupported input_type:", dtype_name(B->dtype_));
        require_dense(A, fn, "A");
        require_dense(B, fn, "B");
        GemmProblem p;
        p.kind = nv ? PK_NVFP4 : PK_MXFP4;
        p.M = M; p.N = N; p.K = Kb * 2;
        p.act    = Operand{A->ptr, M, Kb, Kb, a_preshuffle ? OPM_TILE16 : OPM_ROWMAJOR};
        p.wgt    = Operand{B->ptr, N, Kb, Kb, OPM_TILE16};
        p.act_sf = scale_operand(ScaleA, SFW_G1250, fn, "ScaleA");
        p.wgt_sf = scale_operand(ScaleB, SFW_G1250, fn, "ScaleB");
        require_dense(out, fn, "out");
        if(!out_fp4 && !out_fp8)
        {
            B200_CHECK(out_scale == nullptr, fn, ": out_scale goes with the fp8 output only");
            B200_CHECK(out->dtype_ == AITER_DTYPE_bf16, fn, ": out must be bf16, packed fp4 or fp8 (got ", dtype_name(out->dtype_), ")");
            B200_CHECK(out->shape[0] == M && out->shape[1] == N, fn, ": the bf16 output must be [M, N]");
            p.out_mode = OUT_BF16;
        }
        else if(out_fp4)
        {
            B200_CHECK(out_scale == nullptr, fn, ": the packed fp4 output takes no out_scale");
            B200_CHECK(out->shape[0] == M && out->shape[1] == N / 2, fn, ": the packed fp4 output must be [M, N/2]");
            p.out_mode = OUT_E2M1;
            p.noscale  = 1;
        }
        else
        {
            require_tensor(out_scale, fn, "out_scale", 2);
            B200_CHECK(is_byte_dtype(out_scale->dtype_), fn, ": out_scale must be e8m0 / uint8");
            B200_CHECK(out->shape[0] == M && out->shape[1] == N, fn, ": the fp8 output must be [M, N]");
            B200_CHECK(static_cast<long long>(out_scale->numel_) >= M * (N / 128), fn, ": out_scale must hold M * N/128 bytes");
            require_dense(out_scale, fn, "out_scale");
            require_same_device(A, out_scale, fn, "out_scale");
            p.out_mode  = OUT_MXFP8;
            p.out_scale = out_scale->ptr;
        }
        require_same_device(A, B, fn, "B");
        require_same_device(A, out, fn, "out");
        p.out    = out->ptr;
        p.ldo    = out->strides[0]; // elements of the output's own type (bf16, or one-byte fp8 / packed fp4)
        p.alpha  = global_scale;
        p.beta   = 0.f;
        p.device = A->device_id;
        p.stream = static_cast<cudaStream_t>(stream);
        p.cfg    = tmp.cfg;
        launch_gemm(p);
    }
}

extern "C" int mxfp4_gemm_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA, aiter_tensor_t* ScaleB,
                              aiter_tensor_t* out, aiter_tensor_t* out_scale, const char* kernelName, int a_preshuffle,
                              void* stream)
{
    return safe_call([&] { run_f4gemm("mxfp4_gemm_asm", false, 1.f, A, B, ScaleA, ScaleB, out, out_scale, kernelName, a_preshuffle, stream); });
}

extern "C" int nvfp4_gemm_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA, aiter_tensor_t* ScaleB,
                              float GlobalScaleA, float GlobalScaleB, aiter_tensor_t* out, aiter_tensor_t* out_scale,
                              const char* kernelName, int a_preshuffle, void* stream)
{
    return safe_call([&] {
        // the reference folds float(gA) * float(gB), a double product, into the fp32 result
        const float g = static_cast<float>(static_cast<double>(GlobalScaleA) * static_cast<double>(GlobalScaleB));
        run_f4gemm("nvfp4_gemm_asm", true, g, A, B, ScaleA, ScaleB, out, out_scale, kernelName, a_preshuffle, stream);
    });
}

// ------------------------------------------------------------------------------------------- MXFP8
static void run_mxfp8(const char* fn, int b_is_fp4, aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA,
                      aiter_tensor_t* ScaleB, aiter_tensor_t* out, const char* kernelName, int a_preshuffle, void* stream)
{
    require_tensor(out, fn, "out", 2);
    B200_CHECK(out->dtype_ == AITER_DTYPE_bf16, fn, " only supports BFloat16 output");
    B200_CHECK(a_preshuffle == 0 || a_preshuffle == 1, fn, " a_preshuffle must be 0 or 1");
    require_tensor(A, fn, "A", 2);
    require_tensor(B, fn, "B", 2);
    const long long M = A->shape[0], N = B->shape[0], K = A->shape[1];
    B200_CHECK(K % 128 == 0, fn, " K must be divisible by 128 (got K=", K, ")");
    B200_CHECK(is_byte_dtype(A->dtype_) && is_byte_dtype(B->dtype_), fn, ": A and B must be 1-byte tensors");
    B200_CHECK(B->shape[1] == (b_is_fp4 ? K / 2 : K), fn, ": B must be [N, ", (b_is_fp4 ? "K/2" : "K"), "]");
    require_dense(A, fn, "A");
    require_dense(B, fn, "B");
    GemmProblem p;
    p.kind = b_is_fp4 ? PK_MXF8F4 : PK_MXFP8;
    p.M = M; p.N = N; p.K = K;
    p.act    = Operand{A->ptr, M, K, K, a_preshuffle ? OPM_A2X128 : OPM_ROWMAJOR};
    p.wgt    = Operand{B->ptr, N, b_is_fp4 ? K / 2 : K, b_is_fp4 ? K / 2 : K, OPM_TILE16};
    p.act_sf = scale_operand(ScaleA, SFW_G1250, fn, "ScaleA");
    p.wgt_sf = scale_operand(ScaleB, SFW_G1250, fn, "ScaleB");
    set_out(p, out, fn, M, N);
    p.device = A->device_id;
    p.stream = static_cast<cudaStream_t>(stream);
    apply_config(p, kernelName, -1, fn);
    launch_gemm(p);
}

extern "C" int mxfp8_mxfp8_gemm_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA, aiter_tensor_t* ScaleB,
                                    aiter_tensor_t* out, const char* kernelName, int a_preshuffle, void* stream)
{
    return safe_call([&] { run_mxfp8("mxfp8_mxfp8_gemm_asm", 0, A, B, ScaleA, ScaleB, out, kernelName, a_preshuffle, stream); });
}

extern "C" int mxfp8_mxfp4_gemm_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA, aiter_tensor_t* ScaleB,
                                    aiter_tensor_t* out, const char* kernelName, int a_preshuffle, void* stream)
{
    return safe_call([&] { run_mxfp8("mxfp8_mxfp4_gemm_asm", 1, A, B, ScaleA, ScaleB, out, kernelName, a_preshuffle, stream); });
}

// ------------------------------------------------------------------------------------------- fp8, fp32 128-block scales
static void run_blockscale(const char* fn, aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                           aiter_tensor_t* w_scale, aiter_tensor_t* Out, int bpreshuffle, void* stream,
                           const char* kernelName = nullptr)
{
    require_tensor(XQ, fn, "XQ", 2);
    require_tensor(WQ, fn, "WQ", 2);
    require_tensor(x_scale, fn, "x_scale", 2);
    require_tensor(w_scale, fn, "w_scale", 2);
    require_tensor(Out, fn, "Out", 2);
    B200_CHECK(is_byte_dtype(XQ->dtype_) && is_byte_dtype(WQ->dtype_), fn, ": XQ and WQ must be fp8 (1-byte) tensors");
    const bool sx8 = (x_scale->dtype_ == AITER_DTYPE_fp8_e8m0 || x_scale->dtype_ == AITER_DTYPE_u8);
    const bool sw8 = (w_scale->dtype_ == AITER_DTYPE_fp8_e8m0 || w_scale->dtype_ == AITER_DTYPE_u8);
    B200_CHECK((x_scale->dtype_ == AITER_DTYPE_fp32 && w_scale->dtype_ == AITER_DTYPE_fp32) || (sx8 && sw8), fn,
               ": scales must both be fp32 or both be e8m0 bytes");
    const int out_mode = plain_out_mode(Out->dtype_);
    B200_CHECK(out_mode >= 0, fn, ": Out must be bf16, fp16 or fp32 (got ", dtype_name(Out->dtype_), ")");
    const long long M = XQ->shape[0], K = XQ->shape[1], N = WQ->shape[0];
    B200_CHECK(WQ->shape[1] == K, fn, ": XQ and WQ disagree on K");
    B200_CHECK(K % 128 == 0, fn, ": K must be a multiple of 128");
    B200_CHECK(Out->shape[0] == M && Out->shape[1] == N && Out->strides[1] == 1, fn, ": Out must be [M, N], row-contiguous");
    B200_CHECK(x_scale->shape[0] == M && x_scale->shape[1] == K / 128, fn, ": x_scale must be [M, K/128]");
    B200_CHECK(w_scale->shape[0] == (N + 127) / 128 && w_scale->shape[1] == K / 128, fn, ": w_scale must be [ceil(N/128), K/128]");
    require_dense(WQ, fn, "WQ");
    require_dense(w_scale, fn, "w_scale");
    require_rows_contiguous(XQ, fn, "XQ");
    BlockScaleProblem p;
    p.M = M; p.N = N; p.K = K;
    p.act = Operand{XQ->ptr, M, K, XQ->strides[0], OPM_ROWMAJOR};
    p.wgt = Operand{WQ->ptr, N, K, K, bpreshuffle ? OPM_TILE16 : OPM_ROWMAJOR};
    p.x_scale = static_cast<const float*>(x_scale->ptr);
    if(bpreshuffle && x_scale->strides[1] == 1 && x_scale->strides[0] == K / 128 && M > 1 && K / 128 > 1)
    {
        // the pre-shuffled-weight path takes x_scale stored K-block-major ([K/128][M] in memory), possibly
        // presented under an [M, K/128] view with contiguous-looking strides (the reference's convention)
        p.xs_stride_m = 1;
        p.xs_stride_k = M;
    }
    else
    {
        p.xs_stride_m = x_scale->strides[0];
        p.xs_stride_k = x_scale->strides[1];
    }
    p.w_scale = static_cast<const float*>(w_scale->ptr);
    p.scales_are_e8m0 = sx8 && sw8;
    // a kernel name from a tuned table: "bs_..." picks one of the fp32-scale kernels and its K split; with e8m0 scales
    // the problem may also run on the MXFP8 kernel family, whose configuration names then apply
    if(kernelName != nullptr && kernelName[0] != 0)
    {
        if(parse_blockscale_name(kernelName, p.variant, p.log2_splitk))
            ;
        else if(p.scales_are_e8m0)
        {
            B200_CHECK(parse_config_name(kernelName, p.cfg), fn, ": not find kernel ", kernelName);
            p.cfg_given = true;
        }
        else
            fail(fn, ": not find kernel ", kernelName);
    }
    p.out      = Out->ptr;
    p.ldo      = Out->strides[0];
    p.out_mode = out_mode;
    p.device   = XQ->device_id;
    p.stream   = static_cast<cudaStream_t>(stream);
    launch_blockscale(p);
}

extern "C" int gemm_a8w8_blockscale(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                                    aiter_tensor_t* Out, int splitK, const char* kernelName, void* stream)
{
    (void)splitK; // the fp32-scale kernels have one configuration; kernelName selects among the MXFP8 ones for e8m0 scales
    return safe_call([&] { run_blockscale("gemm_a8w8_blockscale", XQ, WQ, x_scale, w_scale, Out, 0, stream, kernelName); });
}
extern "C" int gemm_a8w8_blockscale_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                                         aiter_tensor_t* Out, int kernelId, int splitK, void* stream)
{
    (void)splitK;
    return safe_call([&] {
        B200_CHECK(kernelId == 0, "gemm_a8w8_blockscale_tune: Kernel id ", kernelId, " not found");
        run_blockscale("gemm_a8w8_blockscale_tune", XQ, WQ, x_scale, w_scale, Out, 0, stream);
    });
}
extern "C" int gemm_a8w8_blockscale_bpreshuffle(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                                aiter_tensor_t* w_scale, aiter_tensor_t* Out, int splitK, const char* kernelName,
                                                void* stream)
{
    (void)splitK;
    return safe_call([&] { run_blockscale("gemm_a8w8_blockscale_bpreshuffle", XQ, WQ, x_scale, w_scale, Out, 1, stream, kernelName); });
}
extern "C" int gemm_a8w8_blockscale_bpreshuffle_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                                     aiter_tensor_t* w_scale, aiter_tensor_t* Out, int kernelId, int splitK, void* stream)
{
    (void)splitK;
    return safe_call([&] {
        B200_CHECK(kernelId == 0, "gemm_a8w8_blockscale_bpreshuffle_tune: Kernel id ", kernelId, " not found");
        run_blockscale("gemm_a8w8_blockscale_bpreshuffle_tune", XQ, WQ, x_scale, w_scale, Out, 1, stream);
    });
}

// The reference binds the same arithmetic under several back-end names (CK, CK-tile, hand-written assembly); here one
// kernel family serves them all, with each name's own argument order.
extern "C" int gemm_a8w8_blockscale_cktile(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                                           aiter_tensor_t* Out, int preshuffleB, int splitK, const char* kernelName, void* stream)
{
    (void)splitK;
    return safe_call([&] { run_blockscale("gemm_a8w8_blockscale_cktile", XQ, WQ, x_scale, w_scale, Out, preshuffleB != 0, stream, kernelName); });
}
extern "C" int gemm_a8w8_blockscale_cktile_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                                                aiter_tensor_t* Out, int kernelId, int splitK, int preshuffleB, void* stream)
{
    (void)splitK;
    return safe_call([&] {
        B200_CHECK(kernelId == 0, "gemm_a8w8_blockscale_cktile_tune: Kernel id ", kernelId, " not found");
        run_blockscale("gemm_a8w8_blockscale_cktile_tune", XQ, WQ, x_scale, w_scale, Out, preshuffleB != 0, stream);
    });
}
extern "C" int gemm_a8w8_blockscale_bpreshuffle_cktile(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                                       aiter_tensor_t* w_scale, aiter_tensor_t* Out, int preshuffleB, const char* kernelName,
                                                       void* stream)
{
    return safe_call([&] { run_blockscale("gemm_a8w8_blockscale_bpreshuffle_cktile", XQ, WQ, x_scale, w_scale, Out, preshuffleB != 0, stream, kernelName); });
}
extern "C" int gemm_a8w8_blockscale_bpreshuffle_cktile_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                                            aiter_tensor_t* w_scale, aiter_tensor_t* Out, int kernelId, int splitK,
                                                            int preshuffleB, void* stream)
{
    (void)splitK;
    return safe_call([&] {
        B200_CHECK(kernelId == 0, "gemm_a8w8_blockscale_bpreshuffle_cktile_tune: Kernel id ", kernelId, " not found");
        run_blockscale("gemm_a8w8_blockscale_bpreshuffle_cktile_tune", XQ, WQ, x_scale, w_scale, Out, preshuffleB != 0, stream);
    });
}
// (XQ, WQ, x_scale, w_scale, out): row-major weight, fp32 scales
extern "C" int flatmm_a8w8_blockscale_asm(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                                          aiter_tensor_t* out, void* stream)
{
    return safe_call([&] { run_blockscale("flatmm_a8w8_blockscale_asm", XQ, WQ, x_scale, w_scale, out, 0, stream); });
}
// (A, B, out, A_scale, B_scale, bias?, splitK, kernelName?, bpreshuffle, zero_bias_buf?): the assembly back-end's order;
// N and K must be multiples of 128 there, and a bias is not part of this library's kernel.
extern "C" int gemm_a8w8_blockscale_bpreshuffle_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* out, aiter_tensor_t* A_scale,
                                                    aiter_tensor_t* B_scale, aiter_tensor_t* bias, int splitK, const char* kernelName,
                                                    int bpreshuffle, aiter_tensor_t* zero_bias_buf, void* stream)
{
    (void)splitK; (void)kernelName; (void)zero_bias_buf;
    return safe_call([&] {
        B200_CHECK(bias == nullptr, "gemm_a8w8_blockscale_bpreshuffle_asm: a bias is not supported by this kernel");
        run_blockscale("gemm_a8w8_blockscale_bpreshuffle_asm", A, B, A_scale, B_scale, out, bpreshuffle != 0, stream);
    });
}

// ------------------------------------------------------------------------------------------- bf16
static void run_bf16(const char* fn, const aiter_tensor_t* A, const aiter_tensor_t* B, const aiter_tensor_t* out,
                     const aiter_tensor_t* bias, int bpreshuffle, const KernelConfig& cfg, void* stream)
{
    // A [.., M, K], B [.., N, K], out [.., M, N]; a leading batch dimension (3-D form) becomes one more tile coordinate
    // of the same launch
    const int a0 = A->ndim - 2;
    B200_CHECK(A->dtype_ == AITER_DTYPE_bf16 && B->dtype_ == AITER_DTYPE_bf16, fn, ": only bf16 inputs are supported (got ",
               dtype_name(A->dtype_), ", ", dtype_name(B->dtype_), ")");
    B200_CHECK(plain_out_mode(out->dtype_) >= 0, fn, ": unsupported output dtype, expected bf16, fp16 or fp32 (got ",
               dtype_name(out->dtype_), ")");
    const long long batch = a0 ? A->shape[0] : 1;
    const long long M = A->shape[a0], K = A->shape[a0 + 1], N = B->shape[a0];
    B200_CHECK(B->shape[a0 + 1] == K, fn, ": A and B disagree on K");
    B200_CHECK(out->shape[a0] == M && out->shape[a0 + 1] == N, fn, ": out must be [M, N]");
    B200_CHECK(A->strides[a0 + 1] == 1 && B->strides[a0 + 1] == 1 && out->strides[a0 + 1] == 1, fn,
               ": tensors must be contiguous along their last dimension");
    B200_CHECK(K % 8 == 0, fn, ": K must be a multiple of 8 for bf16 (16-byte rows)");
    GemmProblem p;
    p.kind = PK_BF16;
    p.M = M; p.N = N; p.K = K;
    p.act = Operand{A->ptr, M, K * 2, A->strides[a0] * 2, OPM_ROWMAJOR};
    if(bpreshuffle)
    {
        B200_CHECK(batch == 1, fn, ": a shuffled weight is not supported with a batch");
        B200_CHECK(B->strides[a0] == K, fn, ": a shuffled weight must be contiguous");
        p.wgt = Operand{B->ptr, N, K * 2, K * 2, OPM_TILE16};
    }
    else
        p.wgt = Operand{B->ptr, N, K * 2, B->strides[a0] * 2, OPM_ROWMAJOR};
    if(batch > 1)
    {
        B200_CHECK(B->shape[0] == batch && out->shape[0] == batch, fn, ": batch mismatch");
        p.batch                  = batch;
        p.act.mode               = OPM_BATCHED;
        p.act.batch              = batch;
        p.act.batch_stride_bytes = A->strides[0] * 2;
        p.wgt.mode               = OPM_BATCHED;
        p.wgt.batch              = batch;
        p.wgt.batch_stride_bytes = B->strides[0] * 2;
        p.out_batch_stride       = out->strides[0];
    }
    p.out      = out->ptr;
    p.ldo      = out->strides[a0];
    p.out_mode = plain_out_mode(out->dtype_);
    if(bias != nullptr)
    {
        B200_CHECK(bias->dtype_ == AITER_DTYPE_bf16 || bias->dtype_ == AITER_DTYPE_fp32, fn, ": bias must be bf16 or fp32");
        // [N] (shared by the batch) or [batch, N]
        const bool per_pair = (bias->ndim == 2 && bias->shape[0] == batch && bias->shape[1] == N && batch > 1);
        B200_CHECK(per_pair || static_cast<long long>(bias->numel_) == N, fn, ": bias must have N elements ([N], or [batch, N])");
        p.bias              = bias->ptr;
        p.bias_is_bf16      = (bias->dtype_ == AITER_DTYPE_bf16);
        p.bias_batch_stride = per_pair ? N : 0;
    }
    p.alpha  = 1.f;
    p.beta   = 1.f;
    p.device = A->device_id;
    p.stream = static_cast<cudaStream_t>(stream);
    p.cfg    = cfg;
    launch_gemm(p);
}

extern "C" int gemm_a16w16_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* out, aiter_tensor_t* semaphore,
                               aiter_tensor_t* bias, int splitK, const char* kernelName, int bpreshuffle, void* stream)
{
    (void)semaphore; // the split-K tickets live in the library's own per-stream workspace
    return safe_call([&] {
        require_tensor(A, "gemm_a16w16_asm", "A", 2);
        require_tensor(B, "gemm_a16w16_asm", "B", 2);
        require_tensor(out, "gemm_a16w16_asm", "out", 2);
        GemmProblem tmp;
        // python passes None as -1; the reference's splitK here is a split count, 0/1 = none
        int l2 = -1;
        if(splitK >= 0)
        {
            l2 = 0;
            while((2 << l2) <= splitK)
                ++l2;
        }
        apply_config(tmp, kernelName, l2, "gemm_a16w16_asm");
        run_bf16("gemm_a16w16_asm", A, B, out, bias, bpreshuffle, tmp.cfg, stream);
    });
}

extern "C" int opus_gemm_a16w16_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* Y, aiter_tensor_t* bias,
                                     int kernelId, int splitK, void* stream)
{
    return safe_call([&] {
        require_tensor(XQ, "opus_gemm_a16w16_tune", "XQ", 3);
        require_tensor(WQ, "opus_gemm_a16w16_tune", "WQ", 3);
        require_tensor(Y, "opus_gemm_a16w16_tune", "Y", 3);
        KernelConfig cfg;
        B200_CHECK(config_from_id(kernelId, cfg), "opus_gemm_a16w16_tune: Kernel id ", kernelId, " not found in a16w16 tune lookup table");
        cfg.log2_splitk = splitK;
        const long long batch = XQ->shape[0];
        B200_CHECK(WQ->shape[0] == batch && Y->shape[0] == batch, "opus_gemm_a16w16_tune: batch mismatch");
        run_bf16("opus_gemm_a16w16_tune", XQ, WQ, Y, bias, 0, cfg, stream);
    });
}

// The CK batched bf16 GEMM's entry points (csrc/ck_batched_gemm_bf16/batched_gemm_bf16.cu:126-148, its _tune twin
// csrc/ck_batched_gemm_bf16/batched_gemm_bf16_tune.cu): Y[b] = XQ[b] WQ[b]^T, all of the batch in one launch.  As there,
// a bias is checked (its dtype must be the output's) and then NOT added - the reference's instances carry no D tensor
// (include/batched_gemm_bf16_common.cuh:165-185) - and its splitK argument is accepted but the K split stays the kernel's
// own choice (KBatch is fixed to 1 there).  Unlike the reference, row and batch strides are free (multiples of 8
// elements), so the [m, b, k] storage of a transposed view is served without a copy.
static void run_batched_bf16(const char* fn, aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* Y, aiter_tensor_t* bias,
                             const KernelConfig& cfg, void* stream)
{
    require_tensor(XQ, fn, "XQ", 3);
    require_tensor(WQ, fn, "WQ", 3);
    require_tensor(Y, fn, "Y", 3);
    B200_CHECK(XQ->dtype_ == AITER_DTYPE_bf16 && WQ->dtype_ == AITER_DTYPE_bf16, fn, ": Weights and activations should both be bf16!");
    B200_CHECK(Y->dtype_ == AITER_DTYPE_bf16 || Y->dtype_ == AITER_DTYPE_fp16, fn, ": the output must be bf16 or fp16 (got ",
               dtype_name(Y->dtype_), ")");
    if(bias != nullptr)
        B200_CHECK(bias->dtype_ == Y->dtype_, fn, ": Out and bias should have the same dtype!");
    B200_CHECK(WQ->shape[0] == XQ->shape[0] && Y->shape[0] == XQ->shape[0], fn, ": batch mismatch");
    run_bf16(fn, XQ, WQ, Y, nullptr, 0, cfg, stream);
}

extern "C" int batched_gemm_bf16(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* out, aiter_tensor_t* bias, int splitK,
                                 void* stream)
{
    (void)splitK;
    return safe_call([&] {
        KernelConfig cfg;
        run_batched_bf16("batched_gemm_bf16", XQ, WQ, out, bias, cfg, stream);
    });
}

extern "C" int batched_gemm_bf16_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* out, int kernelId, int splitK,
                                      void* stream)
{
    return safe_call([&] {
        KernelConfig cfg;
        B200_CHECK(config_from_id(kernelId, cfg), "batched_gemm_bf16_tune: Kernel id ", kernelId, " not found");
        B200_CHECK(splitK >= 0 && splitK <= 8, "batched_gemm_bf16_tune: splitK is log2 of the K split, 0..8");
        cfg.log2_splitk = splitK;
        run_batched_bf16("batched_gemm_bf16_tune", XQ, WQ, out, nullptr, cfg, stream);
    });
}

// one matrix of a [batch, rows, cols] tensor as a 2-D tensor descriptor
static aiter_tensor_t batch_slice(const aiter_tensor_t* t, long long b, int elem_bytes)
{
    aiter_tensor_t s = *t;
    s.ptr        = static_cast<char*>(t->ptr) + b * t->strides[0] * elem_bytes;
    s.ndim       = 2;
    s.shape[0]   = t->shape[1];
    s.shape[1]   = t->shape[2];
    s.strides[0] = t->strides[1];
    s.strides[1] = t->strides[2];
    s.numel_     = static_cast<size_t>(t->shape[1] * t->shape[2]);
    return s;
}

extern "C" int opus_gemm(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* Y, aiter_tensor_t* group_layout,
                         aiter_tensor_t* x_scale, aiter_tensor_t* w_scale, aiter_tensor_t* bias, void* stream)
{
    return safe_call([&] {
        B200_CHECK(group_layout == nullptr, "opus_gemm: grouped layouts are not built");
        require_tensor(XQ, "opus_gemm", "XQ", 3);
        require_tensor(WQ, "opus_gemm", "WQ", 3);
        require_tensor(Y, "opus_gemm", "Y", 3);
        const long long batch = XQ->shape[0];
        B200_CHECK(WQ->shape[0] == batch && Y->shape[0] == batch, "opus_gemm: batch mismatch");
        if(XQ->dtype_ == AITER_DTYPE_fp8)
        {
            // the reference's a8w8_scale pipeline (csrc/opus_gemm/opus_gemm.cu:153-186): fp8 operands, fp32 scales per
            // (row, 128 of K) and per 128 x 128 weight block, fp32 output, no bias; here the fp32-blockscale kernels serve it,
            // one launch per matrix of the batch
            B200_CHECK(x_scale != nullptr && w_scale != nullptr, "opus_gemm: the fp8 form needs x_scale and w_scale (the unscaled a8w8 pipeline is not built)");
            B200_CHECK(bias == nullptr, "opus_gemm: bias is not supported on a8w8 / a8w8_scale paths");
            B200_CHECK(Y->dtype_ == AITER_DTYPE_fp32, "opus_gemm a8w8_scale only supports fp32 output");
            require_tensor(x_scale, "opus_gemm", "x_scale", 3);
            require_tensor(w_scale, "opus_gemm", "w_scale", 3);
            B200_CHECK(x_scale->shape[0] == batch && w_scale->shape[0] == batch, "opus_gemm: scale batch mismatch");
            for(long long b = 0; b < batch; ++b)
            {
                aiter_tensor_t x = batch_slice(XQ, b, 1), w = batch_slice(WQ, b, 1), y = batch_slice(Y, b, 4);
                aiter_tensor_t xs = batch_slice(x_scale, b, 4), ws = batch_slice(w_scale, b, 4);
                run_blockscale("opus_gemm", &x, &w, &xs, &ws, &y, 0, stream);
            }
            return;
        }
        B200_CHECK(x_scale == nullptr && w_scale == nullptr, "opus_gemm: scales go with fp8 operands only");
        KernelConfig cfg;
        run_bf16("opus_gemm", XQ, WQ, Y, bias, 0, cfg, stream);
    });
}

extern "C" int opus_gemm_workspace_init(void) { return 0; }

// ------------------------------------------------------------------------------------------- misc
static constexpr int next_pow2(unsigned int v)
{
    if(v <= 1)
        return 1;
    return 1 << (CHAR_BIT * sizeof(v) - __builtin_clz(v - 1));
}

extern "C" int getPaddedM(int M, int N, int K, int gl)
{
    (void)K;
    int padded = M;
    if(gl == 0)
    {
        const int g = M <= 256 ? 16 : M <= 1024 ? 32 : M <= 4096 ? 64 : 128;
        padded      = (M + g - 1) / g * g;
    }
    else if(gl == 1)
        padded = (M > 8192 && N > 4096) ? 8192 : next_pow2(static_cast<unsigned int>(M));
    return padded;
}

extern "C" int aiter_ctypes_abi_version(void) { return 2; }
extern "C" const char* aiter_get_last_error(void) { return g_last_error.empty() ? nullptr : g_last_error.c_str(); }
extern "C" void aiter_clear_last_error(void) { g_last_error.clear(); }

extern "C" int aiter_b200_device_status(int device, unsigned int out_words[4])
{
    return safe_call([&] { read_device_status(device, out_words); });
}
extern "C" int aiter_b200_debug_wait_control(int device, unsigned long long limit_ns, int withhold_scales)
{
    return safe_call([&] { set_wait_control(device, limit_ns, withhold_scales); });
}
extern "C" const char* aiter_b200_kernel_list(void) { return kernel_menu_text(); }
extern "C" const char* aiter_b200_heuristic_name(int kind, int M, int N, int K, int* log2_splitk)
{
    KernelConfig cfg;
    int sms = 148;
    try
    {
        int dev = 0;
        if(cudaGetDevice(&dev) == cudaSuccess)
            sms = device_sm_count(dev);
    }
    catch(...)
    {
        cudaGetLastError();
    }
    choose_config(kind, M, N, K, sms, cfg);
    if(log2_splitk != nullptr)
        *log2_splitk = cfg.log2_splitk;
    g_heuristic_name = config_name(cfg);
    return g_heuristic_name.c_str();
}
extern "C" unsigned long long aiter_b200_launch_count(void) { return launch_count(); }

// ------------------------------------------------------------------------------------------- dynamic 1x32 MX quantisation
extern "C" int dynamic_per_group_scaled_quant(aiter_tensor_t* out, aiter_tensor_t* input, aiter_tensor_t* scales, int group_size,
                                              int shuffle_scale, aiter_tensor_t* num_rows, int num_rows_factor, void* stream)
{
    return safe_call([&] {
        const char* fn = "dynamic_per_group_scaled_quant";
        require_tensor(out, fn, "out", 2);
        require_tensor(input, fn, "input", 2);
        B200_CHECK(scales != nullptr && scales->device_id >= 0 && scales->ptr != nullptr, fn, ": scales must be a GPU tensor");
        B200_CHECK(group_size == 32, fn, ": only group_size 32 (MX blocks) is built, got ", group_size);
        B200_CHECK(num_rows == nullptr && num_rows_factor == 1, fn, ": num_rows / num_rows_factor (MoE row masks) are not built");
        B200_CHECK(shuffle_scale >= 0 && shuffle_scale <= 2, fn, ": shuffle_scale must be 0 (plain), 1 (e8m0_shuffle) or 2 ((m/32,k/4,32,4))");
        B200_CHECK(input->dtype_ == AITER_DTYPE_bf16 || input->dtype_ == AITER_DTYPE_fp16, fn, ": input must be bf16 or fp16, got ",
                   dtype_name(input->dtype_));
        const bool fp4 = (out->dtype_ == AITER_DTYPE_fp4x2 || out->dtype_ == AITER_DTYPE_u8);
        B200_CHECK(fp4 || out->dtype_ == AITER_DTYPE_fp8, fn, ": out must be fp4x2 / uint8 (MXFP4) or fp8 (MXFP8), got ", dtype_name(out->dtype_));
        B200_CHECK(scales->dtype_ == AITER_DTYPE_fp8_e8m0 || scales->dtype_ == AITER_DTYPE_u8, fn,
                   ": only e8m0 byte scales are built (fp32 scales: use the torch path), got ", dtype_name(scales->dtype_));
        const long long M = input->shape[0], K = input->shape[1];
        B200_CHECK(M > 0 && K > 0 && K % 32 == 0, fn, ": input must be [M, K] with K a multiple of 32");
        require_rows_contiguous(input, fn, "input");
        require_rows_contiguous(out, fn, "out");
        B200_CHECK(input->strides[0] % 8 == 0 && (reinterpret_cast<uintptr_t>(input->ptr) & 15) == 0, fn,
                   ": input rows must start on 16-byte boundaries");
        B200_CHECK(out->shape[0] == M && out->shape[1] == (fp4 ? K / 2 : K), fn, ": out must be [M, ", (fp4 ? "K/2" : "K"), "]");
        B200_CHECK((reinterpret_cast<uintptr_t>(out->ptr) & 7) == 0 && out->strides[0] % 8 == 0, fn, ": out rows must start on 8-byte boundaries");
        const long long kblocks = K / 32;
        B200_CHECK(scales->ndim == 2 && (scales->strides[1] == 1 || scales->shape[1] == 1) && scales->strides[0] == scales->shape[1], fn,
                   ": scales must be a dense 2-D tensor");
        QuantParams prm{};
        prm.layout = shuffle_scale;
        if(shuffle_scale == QSL_E8M0_SHUFFLE)
        {
            B200_CHECK(scales->shape[0] >= (M + 31) / 32 * 32 && scales->shape[1] >= (kblocks + 7) / 8 * 8 && scales->shape[1] % 8 == 0, fn,
                       ": shuffled scales must be [>= pad32(M), pad8(K/32)] (the reference allocates [pad256(M), pad8(K/32)])");
            B200_CHECK((reinterpret_cast<uintptr_t>(scales->ptr) & 7) == 0, fn, ": scales must be 8-byte aligned");
        }
        else if(shuffle_scale == QSL_M32K4)
        {
            B200_CHECK(K % 128 == 0, fn, ": the (m/32,k/4,32,4) scale layout needs K % 128 == 0");
            B200_CHECK(scales->shape[0] >= (M + 31) / 32 * 32 && scales->shape[1] == kblocks, fn, ": scales must be [pad32(M), K/32]");
            B200_CHECK((reinterpret_cast<uintptr_t>(scales->ptr) & 7) == 0, fn, ": scales must be 8-byte aligned");
        }
        else
            B200_CHECK(scales->shape[0] >= M && scales->shape[1] >= kblocks, fn, ": scales must be [M, K/32]");
        prm.in         = input->ptr;
        prm.in_ld      = input->strides[0];
        prm.out        = static_cast<uint8_t*>(out->ptr);
        prm.out_ld     = out->strides[0];
        prm.scale      = static_cast<uint8_t*>(scales->ptr);
        prm.M          = M;
        prm.kblocks    = static_cast<int>(kblocks);
        prm.scale_cols = static_cast<int>(scales->shape[1]);
        int prev = 0;
        B200_CUDA(cudaGetDevice(&prev));
        if(prev != input->device_id)
            B200_CUDA(cudaSetDevice(input->device_id));
        launch_quant_mx(prm, fp4, input->dtype_ == AITER_DTYPE_bf16, static_cast<cudaStream_t>(stream));
        const cudaError_t e = cudaGetLastError();
        if(prev != input->device_id)
            cudaSetDevice(prev);
        B200_CHECK(e == cudaSuccess, fn, ": launch failed: ", cudaGetErrorString(e));
        count_launch();
    });
}
