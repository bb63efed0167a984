// Dynamic 1x32 MX quantisation of activations: bf16 / fp16 [M, K] -> MXFP4 (packed e2m1) or MXFP8 (e4m3) data
// plus one UE8M0 scale byte per 32 elements, written directly in the layout the GEMM consumes.
//
// Arithmetic (bit-exact with the reference's torch path, aiter/ops/quant.py:157-204 and :272-315):
//   amax  = max |x| over the 32-block (fp32)
//   byte  = biased exponent of (amax / max_pos), +1 if any mantissa bit is set (RoundUp), true fp32 division
//   q     = x / 2^(byte-127)           (byte 0 -> 2^-127); done as an exact multiplication by the reciprocal
//   e2m1: round to nearest, ties to the even code, saturate at 6, sign kept on zero;  e4m3: round to nearest even
//
// Work split: one warp per tile of 32 rows x 8 blocks (256 elements of K).  A row of the tile is 512 contiguous
// bytes of input: each lane loads 16 bytes (8 elements), the 4 lanes of a block share their maximum by shuffles,
// every lane converts its 8 elements and the warp writes 128 (fp4) or 256 (fp8) contiguous bytes per row.  The
// tile's 256 scale bytes are exactly one 256-byte chunk of the e8m0_shuffle layout (and two adjacent 128-byte
// chunks of the (m/32, k/4, 32, 4) layout): they are collected in shared memory and stored with two coalesced
// 128-byte stores.  HBM-bound: 2 bytes read + 0.5 / 1 byte written per element, scales 1/32 byte.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cstdint>

namespace b200 {

enum QuantScaleLayout : int { QSL_PLAIN = 0, QSL_E8M0_SHUFFLE = 1, QSL_M32K4 = 2 };

struct QuantParams
{
    const void* in;
    long long in_ld;     // elements between input rows
    uint8_t* out;
    long long out_ld;    // bytes between output rows
    uint8_t* scale;
    long long M;
    int kblocks;         // K / 32
    int scale_cols;      // columns of the scale array (plain: its row pitch; e8m0_shuffle: padded to 8)
    int layout;
};

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v)
{
    return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half v)
{
    return __half2float(v);
}

// Largest magnitude of eight 16-bit floats (bf16 or fp16) as its bit pattern: for non-negative floats the integer order of
// the patterns is the order of the values, infinity sorts above every finite value and NaN above infinity, so the
// unsigned maximum of the sign-less patterns IS the maximum, with a NaN surviving by itself (fmaxf would drop it).
// Two values per instruction (unsigned halfword maximum).
__device__ __forceinline__ uint32_t amax_bits16x8(const uint4& raw)
{
    const uint32_t a = __vmaxu2(raw.x & 0x7FFF7FFFu, raw.y & 0x7FFF7FFFu);
    const uint32_t b = __vmaxu2(raw.z & 0x7FFF7FFFu, raw.w & 0x7FFF7FFFu);
    const uint32_t c = __vmaxu2(a, b);
    return max(c & 0xFFFFu, c >> 16);
}
template <typename T>
__device__ __forceinline__ float bits16_to_f32(uint32_t bits);
template <>
__device__ __forceinline__ float bits16_to_f32<__nv_bfloat16>(uint32_t bits)
{
    return __uint_as_float(bits << 16);
}
template <>
__device__ __forceinline__ float bits16_to_f32<__half>(uint32_t bits)
{
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits)));
}

// SMALL (few tiles, e.g. a decode batch): the eight warps of a CTA share ONE tile, four rows each, so that every load
// of the tile is in flight at once and the kernel lasts about one memory round trip instead of eight.
template <typename T, bool FP4, bool SMALL>
__global__ void __launch_bounds__(256) quant_mx_kernel(const QuantParams prm)
{
    __shared__ __align__(16) uint8_t sf_tile[SMALL ? 1 : 8][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles       = (prm.kblocks + 7) / 8;
    const long long m_tiles = (prm.M + 31) / 32;
    const long long tile    = SMALL ? static_cast<long long>(blockIdx.x) : static_cast<long long>(blockIdx.x) * 8 + warp;
    if(tile >= m_tiles * k_tiles)
        return; // (SMALL: the grid has exactly one CTA per tile, nobody leaves before the barrier below)
    const long long tm = tile / k_tiles;
    const int tk       = static_cast<int>(tile % k_tiles);
    const int blk      = tk * 8 + (lane >> 2);        // this lane's 32-block along K
    const bool blk_ok  = blk < prm.kblocks;
    const float max_pos = FP4 ? 6.0f : 448.0f;
    uint8_t* sf = sf_tile[SMALL ? 0 : warp];
    const int r_begin = SMALL ? warp * 4 : 0, r_end = SMALL ? warp * 4 + 4 : 32;
    const T* in = static_cast<const T*>(prm.in);

    // Rows go through in groups of four; the next group's loads are issued before the current group is converted, so
    // every lane keeps 4 to 8 sixteen-byte loads in flight.
    const long long col_off = static_cast<long long>(tk) * 256 + lane * 8;
    auto load_row = [&](int r) {
        const long long row = tm * 32 + r;
        uint4 raw           = make_uint4(0, 0, 0, 0);
        if(blk_ok && row < prm.M)
            raw = __ldg(reinterpret_cast<const uint4*>(in + row * prm.in_ld + col_off));
        return raw;
    };
    uint4 next[4];
#pragma unroll
    for(int i = 0; i < 4; ++i)
        next[i] = load_row(r_begin + i);
#pragma unroll 1
    for(int r0 = r_begin; r0 < r_end; r0 += 4)
    {
        uint4 cur[4];
#pragma unroll
        for(int i = 0; i < 4; ++i)
            cur[i] = next[i];
        if(r0 + 4 < r_end)
        {
#pragma unroll
            for(int i = 0; i < 4; ++i)
                next[i] = load_row(r0 + 4 + i);
        }
#pragma unroll
        for(int u = 0; u < 4; ++u)
        {
            const int r     = r0 + u;
            const uint4 raw = cur[u];
            const long long row = tm * 32 + r;
            const bool ok       = blk_ok && row < prm.M;
            const T* e = reinterpret_cast<const T*>(&raw);
            float v[8];
#pragma unroll
            for(int i = 0; i < 8; ++i)
                v[i] = to_f32<T>(e[i]);
            // the block's largest magnitude, NaN included, on the 16-bit patterns; the four lanes of a block share it
            uint32_t ab = amax_bits16x8(raw);
            ab          = max(ab, __shfl_xor_sync(0xffffffffu, ab, 1));
            ab          = max(ab, __shfl_xor_sync(0xffffffffu, ab, 2));
            const float amax  = bits16_to_f32<T>(ab);
            const uint32_t qb = __float_as_uint(__fdiv_rn(amax, max_pos));
            const uint32_t ex = (qb >> 23) & 0xFFu;
            const uint32_t byte = ex + (((qb & 0x7FFFFFu) != 0u && ex < 0xFFu) ? 1u : 0u);
            // 1 / 2^(byte-127), exact: multiplying by it rounds like the reference's division by the scale
            // (byte 0 stands for 2^-127, byte 254 needs the denormal 2^-127, byte 255 is NaN)
            const float rscale = __uint_as_float(byte == 0xFFu ? 0x7F800001u : (byte == 254u ? 0x00400000u : ((254u - byte) << 23)));
            if(FP4)
            {
                // cvt.rn.satfinite.e2m1x2.f32: nearest, ties to even, saturating at 6, sign kept on zero; low nibble = even element
                uint32_t packed = 0;
#pragma unroll
                for(int i = 0; i < 4; ++i)
                    packed |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(make_float2(v[2 * i] * rscale, v[2 * i + 1] * rscale), __NV_E2M1,
                                                                             cudaRoundNearest))
                              << (8 * i);
                if(ok)
                    *reinterpret_cast<uint32_t*>(prm.out + row * prm.out_ld + static_cast<long long>(tk) * 128 + lane * 4) = packed;
            }
            else
            {
                uint32_t w[2];
#pragma unroll
                for(int h = 0; h < 2; ++h)
                {
                    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
                        make_float2(v[4 * h] * rscale, v[4 * h + 1] * rscale), __NV_SATFINITE, __NV_E4M3);
                    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
                        make_float2(v[4 * h + 2] * rscale, v[4 * h + 3] * rscale), __NV_SATFINITE, __NV_E4M3);
                    w[h] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
                }
                if(ok)
                    *reinterpret_cast<uint2*>(prm.out + row * prm.out_ld + static_cast<long long>(tk) * 256 + lane * 8) = make_uint2(w[0], w[1]);
            }
            // one lane per block files the scale byte at its place inside the tile's 256-byte chunk
            if((lane & 3) == 0)
            {
                const int kb = lane >> 2; // block within the tile, 0..7
                const uint8_t b = ok ? static_cast<uint8_t>(byte) : static_cast<uint8_t>(prm.layout == QSL_M32K4 ? 0x7F : 0);
                int pos;
                if(prm.layout == QSL_E8M0_SHUFFLE)
                    pos = (kb & 3) * 64 + (r & 15) * 4 + (kb >> 2) * 2 + (r >> 4);
                else if(prm.layout == QSL_M32K4)
                    pos = (kb >> 2) * 128 + r * 4 + (kb & 3);
                else
                    pos = r * 8 + kb;
                sf[pos] = b;
            }
        }
    }
    if(SMALL)
    {
        __syncthreads();
        if(warp != 0)
            return;
    }
    else
        __syncwarp();
    if(prm.layout == QSL_E8M0_SHUFFLE)
    {
        // chunk of (row group tm, K tile tk): byte offset (tm * scale_cols) * 32 + tk * 256
        uint8_t* dst = prm.scale + (tm * prm.scale_cols) * 32 + static_cast<long long>(tk) * 256;
        reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(sf)[lane];
    }
    else if(prm.layout == QSL_M32K4)
    {
        // two 128-byte chunks, K atoms 2 tk and 2 tk + 1 (the second only if it exists)
        const int atoms = prm.kblocks / 4;
        uint8_t* dst    = prm.scale + (tm * atoms + 2LL * tk) * 128;
        const int valid = min(2, atoms - 2 * tk) * 128;
        if(lane * 8 < valid)
            reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(sf)[lane];
    }
    else
    {
        // plain [M][K/32]: 8 bytes per row of the tile
        const long long row = tm * 32 + lane;
        if(row < prm.M)
        {
            uint8_t* dst = prm.scale + row * prm.scale_cols + tk * 8;
            const int n  = min(8, prm.kblocks - tk * 8);
            for(int i = 0; i < n; ++i)
                dst[i] = sf[lane * 8 + i];
        }
    }
}

inline void launch_quant_mx(const QuantParams& prm, bool fp4, bool input_is_bf16, cudaStream_t stream)
{
    const long long tiles = ((prm.M + 31) / 32) * ((prm.kblocks + 7) / 8);
    if(tiles <= 2048)
    {
        // few tiles: one CTA per tile
        const unsigned blocks = static_cast<unsigned>(tiles);
        if(fp4 && input_is_bf16)
            quant_mx_kernel<__nv_bfloat16, true, true><<<blocks, 256, 0, stream>>>(prm);
        else if(fp4)
            quant_mx_kernel<__half, true, true><<<blocks, 256, 0, stream>>>(prm);
        else if(input_is_bf16)
            quant_mx_kernel<__nv_bfloat16, false, true><<<blocks, 256, 0, stream>>>(prm);
        else
            quant_mx_kernel<__half, false, true><<<blocks, 256, 0, stream>>>(prm);
        return;
    }
    const unsigned blocks = static_cast<unsigned>((tiles + 7) / 8);
    if(fp4 && input_is_bf16)
        quant_mx_kernel<__nv_bfloat16, true, false><<<blocks, 256, 0, stream>>>(prm);
    else if(fp4)
        quant_mx_kernel<__half, true, false><<<blocks, 256, 0, stream>>>(prm);
    else if(input_is_bf16)
        quant_mx_kernel<__nv_bfloat16, false, false><<<blocks, 256, 0, stream>>>(prm);
    else
        quant_mx_kernel<__half, false, false><<<blocks, 256, 0, stream>>>(prm);
}

} // namespace b200
