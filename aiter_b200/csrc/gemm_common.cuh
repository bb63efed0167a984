// Shared pieces of the tcgen05 GEMM kernels: enums, status codes, bounded waits, small device helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <type_traits>
#include "ptx.cuh"

// Timestamp probes of the single-thread roles, compiled in only with -DAITER_B200_TRACING (a development aid: a
// probe in a loop that one thread runs per K tile costs that loop several cycles per dependent instruction).
#ifdef AITER_B200_TRACING
#define B200_TRACE(...) __VA_ARGS__
#else
#define B200_TRACE(...)
#endif

namespace b200 {

enum GemmKind : int
{
    KIND_BF16   = 0,
    KIND_MXF8   = 1,
    KIND_MXF4   = 2,
    KIND_MXF8F4 = 3, // e4m3 activations x e2m1 weights
    KIND_NVF4   = 4, // e2m1 x e2m1 with one e4m3 scale per 16 elements (NVFP4); wire scale tiles are 32 rows x 8 bytes
};
enum OperandMode : int { OPM_ROWMAJOR = 0, OPM_TILE16 = 1, OPM_A2X128 = 2, OPM_BATCHED = 4 /* row-major, one matrix per batch entry */ };
enum SfWire : int { SFW_NONE = 0, SFW_G1250 = 1, SFW_E8M0_SHUFFLE = 2 };

constexpr int kMaxStages  = 8;
constexpr int kTileP      = 128;
constexpr int kTileKBytes = 128;
constexpr int kNumThreads = 224;
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull; // 1 s per wait unless the host lowers it

// Per-device controls of the bounded waits, in constant memory so that a test can shorten the limit and make a
// wait run out on purpose without rebuilding.  The host writes it (launch.cu: device set-up, and the
// aiter_b200_debug_wait_control entry point); kernels read it only on the slow path of a wait.
struct WaitControl
{
    unsigned long long limit_ns;  // wall-time bound of every in-kernel wait
    unsigned int* host_mirror;    // pinned, device-mapped host word that receives the first failure code (may be null)
    unsigned int withhold_scales; // test hook: the raw-scale producer of the persistent kernel issues nothing, so
                                  // the waits of the roles behind it run out after limit_ns
};
static __constant__ WaitControl c_wait_ctl = {kWaitLimitNs, nullptr, 0u};

// status codes (word 0 of the status buffer); words 1..3 carry blockIdx / iteration detail
constexpr uint32_t kParkNs = 20000; // longest single park of a waiting thread; the wall-time bound is checked between parks
constexpr uint32_t ST_TIMEOUT_PRODUCER = 0x101;
constexpr uint32_t ST_TIMEOUT_MMA_FULL = 0x102;
constexpr uint32_t ST_TIMEOUT_MMA_SF   = 0x103;
constexpr uint32_t ST_TIMEOUT_SFWARP   = 0x104;
constexpr uint32_t ST_TIMEOUT_EPILOGUE = 0x105;
constexpr uint32_t ST_TIMEOUT_DRAIN    = 0x106;

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");
    return t;
}

// Wait for an mbarrier phase for at most c_wait_ctl.limit_ns of wall time.  Returns false when the wait
// expired (first expiry records `code` in the status words and raises the CTA abort flag) or when
// another role of this CTA already aborted.
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                             unsigned int* status, uint32_t code, uint32_t detail)
{
    if(mbar_try_wait(bar, parity))
        return true;
    const uint64_t t0    = global_timer_ns();
    const uint64_t limit = c_wait_ctl.limit_ns;
    for(;;)
    {
        if(mbar_try_wait_parked(bar, parity, kParkNs))
            return true;
        if(*abort_flag)
            return false;
        if(global_timer_ns() - t0 > limit)
            break;
    }
    *abort_flag = 1;
    if(atomicCAS(status, 0u, code) == 0u)
    {
        status[1] = blockIdx.x | (blockIdx.y << 16);
        status[2] = blockIdx.z;
        status[3] = detail;
        // the host checks this word before every launch, so the failure surfaces at the caller's next call
        unsigned int* mirror = c_wait_ctl.host_mirror;
        if(mirror != nullptr)
        {
            *reinterpret_cast<volatile unsigned int*>(mirror) = code;
            __threadfence_system();
        }
    }
    return false;
}

// prmt in its default mode: selector nibble bit 3 set = fill the byte with the selected byte's sign bit
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// 8 packed e2m1 codes (one 32-bit word, element n in nibble n) -> 8 e4m3 bytes (exact: every e2m1 value
// is an e4m3 value).  Magnitude by table look-up (prmt on the 3-bit magnitude codes); the sign bits sit at bit 7
// of the bytes of w (odd codes) and of w << 4 (even codes), from where a sign-replicating prmt spreads them over
// whole bytes and one and-or keeps bit 7.
__device__ __forceinline__ void e2m1x8_to_e4m3x8(uint32_t w, uint32_t& lo, uint32_t& hi)
{
    constexpr uint32_t kLutLo = 0x3C383000u; // 0, 0.5, 1, 1.5
    constexpr uint32_t kLutHi = 0x4C484440u; // 2, 3, 4, 6
    const uint32_t mag = w & 0x77777777u;
    const uint32_t x   = w << 4;
    const uint32_t s_lo = prmt_b32(w, x, 0x9D8Cu); // codes 0..3: bytes x.0, w.0, x.1, w.1, sign-replicated
    const uint32_t s_hi = prmt_b32(w, x, 0xBFAEu); // codes 4..7: bytes x.2, w.2, x.3, w.3
    lo = prmt_b32(kLutLo, kLutHi, mag) | (s_lo & 0x80808080u);
    hi = prmt_b32(kLutLo, kLutHi, mag >> 16) | (s_hi & 0x80808080u);
}

__device__ __forceinline__ void issue_operand_load(int mode, uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                   int row0, int k_iter)
{
    if(mode == OPM_ROWMAJOR)
        tma_load_2d(dst, map, bar, k_iter * kTileKBytes, row0);
    else if(mode == OPM_TILE16)
        tma_load_3d(dst, map, bar, 0, row0 >> 4, k_iter * (kTileKBytes / 16));
    else
        tma_load_4d(dst, map, bar, 0, 0, row0 >> 1, k_iter);
}

__device__ __forceinline__ float load_bias(const void* bias, int is_bf16, int idx)
{
    return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[idx])
                   : __ldg(static_cast<const float*>(bias) + idx);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Output element types of the GEMM epilogues.
enum OutMode : int
{
    OUT_BF16  = 0,
    OUT_F16   = 1,
    OUT_F32   = 2,
    OUT_E2M1  = 3, // packed e2m1, two per byte, no scale (the reference's gemm_a4w4o4)
    OUT_MXFP8 = 4, // e4m3 data + one UE8M0 scale per 128 output columns (the reference's gemm_a4w4o8)
};

__device__ __forceinline__ uint32_t pack_f16x2(float a, float b)
{
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
// two fp32 values -> two 16-bit outputs (bf16, or fp16 when f16 is set) in one word
__device__ __forceinline__ uint32_t pack_out16x2(float a, float b, bool f16) { return f16 ? pack_f16x2(a, b) : pack_bf16x2(a, b); }
__device__ __forceinline__ uint16_t cvt_out16(float a, bool f16)
{
    return f16 ? __half_as_ushort(__float2half_rn(a)) : __bfloat16_as_ushort(__float2bfloat16_rn(a));
}
// N consecutive outputs of one row, starting at element index `at`; `valid` of them lie inside the matrix.  vec: the row
// start is 16-byte aligned (16-byte stores for every whole group of valid elements)
template <int N>
__device__ __forceinline__ void store_row(void* base, int mode, size_t at, const float (&v)[N], int valid, bool vec)
{
    // (a ragged last tile keeps its vector stores for the whole groups that are valid: scalar stores of a row segment
    // go out as one 2- or 4-byte transaction per lane and measured +11 us on 512 x 576 x 7168)
    if(mode == OUT_F32)
    {
        float* dst = static_cast<float*>(base) + at;
        if(vec)
        {
#pragma unroll
            for(int i = 0; i < N; i += 4)
            {
                if(i + 4 <= valid)
                    *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                else
                {
#pragma unroll
                    for(int e = 0; e < 4; ++e)
                        if(i + e < valid)
                            dst[i + e] = v[i + e];
                }
            }
        }
        else
        {
#pragma unroll
            for(int i = 0; i < N; ++i)
                if(i < valid)
                    dst[i] = v[i];
        }
    }
    else
    {
        const bool f16 = (mode == OUT_F16);
        uint16_t* dst  = static_cast<uint16_t*>(base) + at;
        if(vec)
        {
#pragma unroll
            for(int i = 0; i < N; i += 8)
            {
                if(i + 8 <= valid)
                    *reinterpret_cast<uint4*>(dst + i) = make_uint4(pack_out16x2(v[i], v[i + 1], f16), pack_out16x2(v[i + 2], v[i + 3], f16),
                                                                    pack_out16x2(v[i + 4], v[i + 5], f16), pack_out16x2(v[i + 6], v[i + 7], f16));
                else
                {
#pragma unroll
                    for(int e = 0; e < 8; ++e)
                        if(i + e < valid)
                            dst[i + e] = cvt_out16(v[i + e], f16);
                }
            }
        }
        else
        {
#pragma unroll
            for(int i = 0; i < N; ++i)
                if(i < valid)
                    dst[i] = cvt_out16(v[i], f16);
        }
    }
}
// one output element of a 16- or 32-bit output array
__device__ __forceinline__ void store_out(void* base, size_t idx, float v, int mode)
{
    if(mode == OUT_F32)
        static_cast<float*>(base)[idx] = v;
    else
        static_cast<uint16_t*>(base)[idx] = cvt_out16(v, mode == OUT_F16);
}


} // namespace b200
