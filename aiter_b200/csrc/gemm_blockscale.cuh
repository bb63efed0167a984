// FP8 x FP8 GEMM with fp32 scales per 128-wide K block: x_scale[M][K/128] (one per activation row and K
// block) and w_scale[N/128][K/128] (one per 128x128 weight block), bf16 output.
//
//   out[m][n] = sum_kb  xs[m][kb] * ws[n/128][kb] * sum_{k in block kb} A[m][k] * B[n][k]
//
// fp32 scales cannot ride the block-scaled MMA (its scales are powers of two), so every K block is
// multiplied unscaled (tcgen05.mma kind::f8f6f4, 4 instructions of K = 32) into one of two TMEM partial
// accumulators, and the 128 epilogue threads (one output row each) promote the finished partial into fp32
// register accumulators with the two scales applied, while the tensor core fills the other partial.
//
// One 128x128 output tile per CTA.  Warps (192 threads): 0 TMA producer, 1 MMA issuer + TMEM owner,
// 2..5 promotion + store.  Every barrier wait is bounded (see bounded_wait).
#pragma once
#include "gemm_common.cuh"

namespace b200 {

constexpr int kBlockScaleThreads = 192;
constexpr int kBsTileN           = 128;

struct BlockScaleParams
{
    int M, N;
    int k_blocks;            // K / 128
    int stages;
    int a_mode, b_mode;      // OperandMode of activations / weights
    const float* x_scale;
    long long xs_stride_m, xs_stride_k; // in elements
    const float* w_scale;    // [ceil(N/128)][k_blocks]
    __nv_bfloat16* out;
    long long ldo;
    unsigned int* status;
};

__host__ __device__ constexpr uint32_t idesc_f8f6f4_e4m3(uint32_t m, uint32_t n)
{
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); // D fp32, A/B e4m3 (format 0), K-major
}

__device__ __forceinline__ void mma_f8f6f4(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(kBlockScaleThreads, 1)
gemm_a8w8_blockscale_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            const BlockScaleParams prm)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const int S              = prm.stages;
    constexpr uint32_t kStageBytes = (kTileP + kBsTileN) * kTileKBytes; // 32 KB
    const uint32_t bar_base  = smem_base + kStageBytes * S;
    auto full_bar       = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar      = [&](int s) { return bar_base + 64u + 8u * s; };
    auto part_full_bar  = [&](int b) { return bar_base + 128u + 8u * b; };
    auto part_empty_bar = [&](int b) { return bar_base + 144u + 8u * b; };
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + kStageBytes * S + 160);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + kStageBytes * S + 164);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kTileP;
    const int col0 = blockIdx.y * kBsTileN;
    const int KB   = prm.k_blocks;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(part_full_bar(b), 1);
            mbar_init(part_empty_bar(b), 4);
        }
        *abort_f = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if(warp == 1)
    {
        tmem_alloc(smem_u32(tmem_ptr_smem), 256);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if(warp == 0)
    {
        if(lane == 0)
        {
            int issued = 0;
            for(int j = 0; j < KB; ++j)
            {
                const int s = j % S;
                if(!bounded_wait(empty_bar(s), ((j / S) & 1) ^ 1, abort_f, prm.status, ST_TIMEOUT_PRODUCER, j))
                    break;
                const uint32_t stage = smem_base + s * kStageBytes;
                mbar_arrive_expect_tx(full_bar(s), kStageBytes);
                issue_operand_load(prm.a_mode, stage, &map_a, full_bar(s), row0, j);
                issue_operand_load(prm.b_mode, stage + kTileP * kTileKBytes, &map_b, full_bar(s), col0, j);
                issued = j + 1;
            }
            if(*abort_f)
                for(int j = issued - 1; j >= 0 && j >= issued - S; --j)
                {
                    const uint64_t t0 = global_timer_ns();
                    while(!mbar_try_wait(full_bar(j % S), (j / S) & 1) && global_timer_ns() - t0 < kWaitLimitNs) {}
                }
        }
    }
    else if(warp == 1)
    {
        if(lane == 0)
        {
            const uint32_t idesc = idesc_f8f6f4_e4m3(kTileP, kBsTileN);
            const bool a_tiled = (prm.a_mode == OPM_TILE16), b_tiled = (prm.b_mode == OPM_TILE16);
            const uint32_t a_lbo = a_tiled ? kTileP * 16u : 16u, a_sbo = a_tiled ? 128u : 1024u, a_lay = a_tiled ? 0u : 2u;
            const uint32_t a_adv = a_tiled ? 2u * kTileP * 16u : 32u;
            const uint32_t b_lbo = b_tiled ? kBsTileN * 16u : 16u, b_sbo = b_tiled ? 128u : 1024u, b_lay = b_tiled ? 0u : 2u;
            const uint32_t b_adv = b_tiled ? 2u * kBsTileN * 16u : 32u;
            bool ok = true;
            for(int j = 0; j < KB && ok; ++j)
            {
                const int s = j % S, b = j & 1;
                ok = bounded_wait(part_empty_bar(b), ((j >> 1) & 1) ^ 1, abort_f, prm.status, ST_TIMEOUT_MMA_SF, j);
                if(ok)
                    ok = bounded_wait(full_bar(s), (j / S) & 1, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, j);
                if(!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t stage = smem_base + s * kStageBytes;
#pragma unroll
                for(int k = 0; k < 4; ++k)
                    mma_f8f6f4(tmem_base + b * kBsTileN, make_smem_desc(stage + k * a_adv, a_lbo, a_sbo, a_lay),
                               make_smem_desc(stage + kTileP * kTileKBytes + k * b_adv, b_lbo, b_sbo, b_lay), idesc, k > 0 ? 1u : 0u);
                tc_commit(empty_bar(s));
                tc_commit(part_full_bar(b));
            }
        }
    }
    else
    {
        // promotion + store: thread = output row
        const int quarter    = warp & 3;
        const int r_local    = quarter * 32 + lane;
        const int row        = row0 + r_local;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const bool row_ok    = row < prm.M;
        const float* xs      = prm.x_scale + static_cast<long long>(row_ok ? row : 0) * prm.xs_stride_m;
        const float* ws      = prm.w_scale + static_cast<long long>(blockIdx.y) * KB;
        float acc[kBsTileN];
#pragma unroll
        for(int i = 0; i < kBsTileN; ++i)
            acc[i] = 0.f;
        bool ok = true;
        float scale_next = (KB > 0) ? __ldg(xs) * __ldg(ws) : 0.f;
        for(int j = 0; j < KB && ok; ++j)
        {
            const int b       = j & 1;
            const float scale = scale_next;
            if(j + 1 < KB)
                scale_next = __ldg(xs + static_cast<long long>(j + 1) * prm.xs_stride_k) * __ldg(ws + j + 1);
            ok = bounded_wait(part_full_bar(b), (j >> 1) & 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, j);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                break;
            tc_fence_after_sync();
#pragma unroll
            for(int c = 0; c < kBsTileN / 32; ++c)
            {
                uint32_t r[32];
                tmem_ld_x32(tlane + b * kBsTileN + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for(int i = 0; i < 32; ++i)
                    acc[c * 32 + i] = fmaf(__uint_as_float(r[i]), scale, acc[c * 32 + i]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
                mbar_arrive(part_empty_bar(b));
        }
        if(ok && row_ok)
        {
            __nv_bfloat16* dst = prm.out + static_cast<size_t>(row) * prm.ldo + col0;
            const bool vec_ok  = ((prm.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(prm.out) & 15) == 0) && (col0 + kBsTileN <= prm.N);
            if(vec_ok)
            {
#pragma unroll
                for(int i = 0; i < kBsTileN; i += 8)
                    *reinterpret_cast<uint4*>(dst + i) = make_uint4(pack_bf16x2(acc[i], acc[i + 1]), pack_bf16x2(acc[i + 2], acc[i + 3]),
                                                                    pack_bf16x2(acc[i + 4], acc[i + 5]), pack_bf16x2(acc[i + 6], acc[i + 7]));
            }
            else
            {
#pragma unroll
                for(int i = 0; i < kBsTileN; ++i)
                    if(col0 + i < prm.N)
                        dst[i] = __float2bfloat16_rn(acc[i]);
            }
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    if(warp == 1)
    {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 256);
    }
}


// ---------------------------------------------------------------------------------------------------------
// Same arithmetic on CTA pairs: a 256 x 256 output tile per pair (cta_group::2).  Every CTA stages its own 128
// rows of A and its own 128 of the tile's 256 rows of B per K block (24 B of operand per 512 cycles of MMA and
// SM less than the 128 x 128 tile moves), the leader issues 256 x 256 x 32 MMAs into one of two 256-column
// TMEM partials, and eight promotion warps per CTA (two per TMEM lane quarter, 128 columns each) fold the
// finished partial into fp32 registers with x_scale[m][kb] * w_scale[n/128][kb].
// Warps (352 threads): 0 TMA producer, 1 MMA issuer (leader) + TMEM owner, 2..9 promotion + store, 10 idle.
constexpr int kBlockScalePairThreads = 352;
constexpr int kBsPairN               = 256;

__device__ __forceinline__ void mma_f8f6f4_2cta(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(kBlockScalePairThreads, 1)
gemm_a8w8_blockscale_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                 const BlockScaleParams prm)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const int S              = prm.stages;
    constexpr uint32_t kStageBytes = 2u * kTileP * kTileKBytes; // 16 KB of A + 16 KB of B per CTA
    const uint32_t bar_base  = smem_base + kStageBytes * S;
    auto full_bar       = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar      = [&](int s) { return bar_base + 64u + 8u * s; };
    auto part_full_bar  = [&](int b) { return bar_base + 128u + 8u * b; };
    auto part_empty_bar = [&](int b) { return bar_base + 144u + 8u * b; };
    const uint32_t drain_bar   = bar_base + 160u;
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + kStageBytes * S + 168);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + kStageBytes * S + 172);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_ctarank();
    const bool leader    = (crank == 0);
    const int pair_x     = blockIdx.x >> 1;                 // 256-row tile index
    const int row0       = (pair_x * 2 + static_cast<int>(crank)) * kTileP;
    const int col0       = blockIdx.y * kBsPairN;
    const int KB         = prm.k_blocks;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            mbar_init(full_bar(s), 2);  // one expect_tx arrival per CTA of the pair
            mbar_init(empty_bar(s), 1);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(part_full_bar(b), 1);
            mbar_init(part_empty_bar(b), 16); // eight promotion warps in each CTA
        }
        mbar_init(drain_bar, 1);
        *abort_f = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if(warp == 10 && lane == 0)
    {
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if(warp == 1)
    {
        tmem_alloc_2cta(smem_u32(tmem_ptr_smem), 512);
        tmem_relinquish_2cta();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if(warp == 0)
    {
        if(lane == 0)
        {
            const uint32_t full0 = map_to_cta(full_bar(0), 0);
            int s = 0;
            uint32_t phase = 0;
            for(int j = 0; j < KB; ++j)
            {
                if(!bounded_wait(empty_bar(s), phase ^ 1u, abort_f, prm.status, ST_TIMEOUT_PRODUCER, j))
                    break;
                const uint32_t stage = smem_base + s * kStageBytes;
                const uint32_t bar   = full0 + 8u * s;
                mbar_arrive_expect_tx_cluster(bar, kStageBytes);
                if(prm.a_mode == OPM_ROWMAJOR)
                    tma_load_2d_pair(stage, &map_a, bar, j * kTileKBytes, row0);
                else
                    tma_load_3d_pair(stage, &map_a, bar, 0, row0 >> 4, j * (kTileKBytes / 16));
                const int brow = col0 + static_cast<int>(crank) * kTileP;
                if(prm.b_mode == OPM_ROWMAJOR)
                    tma_load_2d_pair(stage + kTileP * kTileKBytes, &map_b, bar, j * kTileKBytes, brow);
                else
                    tma_load_3d_pair(stage + kTileP * kTileKBytes, &map_b, bar, 0, brow >> 4, j * (kTileKBytes / 16));
                if(++s == S)
                {
                    s = 0;
                    phase ^= 1u;
                }
            }
            if(*abort_f)
            {
                const uint64_t t0 = global_timer_ns();
                while(global_timer_ns() - t0 < 200000ull) {}
            }
        }
    }
    else if(warp == 1)
    {
        if(lane == 0 && leader)
        {
            const uint32_t idesc = idesc_f8f6f4_e4m3(2 * kTileP, kBsPairN);
            const bool a_tiled = (prm.a_mode == OPM_TILE16), b_tiled = (prm.b_mode == OPM_TILE16);
            const uint32_t a_lbo = a_tiled ? kTileP * 16u : 16u, a_sbo = a_tiled ? 128u : 1024u, a_lay = a_tiled ? 0u : 2u;
            const uint32_t a_step = (a_tiled ? 2u * kTileP * 16u : 32u) >> 4;
            const uint32_t b_lbo = b_tiled ? kTileP * 16u : 16u, b_sbo = b_tiled ? 128u : 1024u, b_lay = b_tiled ? 0u : 2u;
            const uint32_t b_step = (b_tiled ? 2u * kTileP * 16u : 32u) >> 4;
            const uint32_t a_hi  = static_cast<uint32_t>(make_smem_desc(0, a_lbo, a_sbo, a_lay) >> 32);
            const uint32_t b_hi  = static_cast<uint32_t>(make_smem_desc(0, b_lbo, b_sbo, b_lay) >> 32);
            const uint32_t a_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base, a_lbo, a_sbo, a_lay));
            const uint32_t b_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base + kTileP * kTileKBytes, b_lbo, b_sbo, b_lay));
            bool ok = true;
            int s = 0;
            uint32_t phase = 0;
            for(int j = 0; j < KB && ok; ++j)
            {
                const int b = j & 1;
                ok = bounded_wait(part_empty_bar(b), ((j >> 1) & 1) ^ 1, abort_f, prm.status, ST_TIMEOUT_MMA_SF, j);
                if(ok)
                    ok = bounded_wait(full_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, j);
                if(!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t a_lo = a_lo0 + s * (kStageBytes >> 4), b_lo = b_lo0 + s * (kStageBytes >> 4);
#pragma unroll
                for(int k = 0; k < 4; ++k)
                    mma_f8f6f4_2cta(tmem_base + b * kBsPairN, pack_u64(a_lo + k * a_step, a_hi), pack_u64(b_lo + k * b_step, b_hi), idesc,
                                    k > 0 ? 1u : 0u);
                tc_commit_2cta(empty_bar(s), 3);
                tc_commit_2cta(part_full_bar(b), 3);
                if(++s == S)
                {
                    s = 0;
                    phase ^= 1u;
                }
            }
            if(!ok)
            {
                tc_commit_2cta(drain_bar, 1);
                const uint64_t t0 = global_timer_ns();
                while(!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < kWaitLimitNs) {}
            }
        }
    }
    else if(warp < 10)
    {
        // promotion + store: thread = output row, 128 of the tile's 256 columns
        const int quarter    = warp & 3;
        const int half       = (warp - 2) >> 2;
        const int r_local    = quarter * 32 + lane;
        const int row        = row0 + r_local;
        const int ccol0      = col0 + half * 128;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 128;
        const bool row_ok    = row < prm.M;
        const float* xs      = prm.x_scale + static_cast<long long>(row_ok ? row : 0) * prm.xs_stride_m;
        const int nblk       = min(ccol0 / 128, (prm.N + 127) / 128 - 1);
        const float* ws      = prm.w_scale + static_cast<long long>(nblk) * KB;
        const uint32_t part_empty_leader = map_to_cta(part_empty_bar(0), 0);
        float acc[128];
#pragma unroll
        for(int i = 0; i < 128; ++i)
            acc[i] = 0.f;
        bool ok = true;
        float scale_next = (KB > 0) ? __ldg(xs) * __ldg(ws) : 0.f;
        for(int j = 0; j < KB && ok; ++j)
        {
            const int b       = j & 1;
            const float scale = scale_next;
            if(j + 1 < KB)
                scale_next = __ldg(xs + static_cast<long long>(j + 1) * prm.xs_stride_k) * __ldg(ws + j + 1);
            ok = bounded_wait(part_full_bar(b), (j >> 1) & 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, j);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                break;
            tc_fence_after_sync();
#pragma unroll
            for(int c = 0; c < 4; ++c)
            {
                uint32_t r[32];
                tmem_ld_x32(tlane + b * kBsPairN + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for(int i = 0; i < 32; ++i)
                    acc[c * 32 + i] = fmaf(__uint_as_float(r[i]), scale, acc[c * 32 + i]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
                mbar_arrive_cluster(part_empty_leader + 8u * b);
        }
        if(ok && row_ok)
        {
            __nv_bfloat16* dst = prm.out + static_cast<size_t>(row) * prm.ldo + ccol0;
            const bool vec_ok  = ((prm.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(prm.out) & 15) == 0) && (ccol0 + 128 <= prm.N);
            if(vec_ok)
            {
#pragma unroll
                for(int i = 0; i < 128; i += 8)
                    *reinterpret_cast<uint4*>(dst + i) = make_uint4(pack_bf16x2(acc[i], acc[i + 1]), pack_bf16x2(acc[i + 2], acc[i + 3]),
                                                                    pack_bf16x2(acc[i + 4], acc[i + 5]), pack_bf16x2(acc[i + 6], acc[i + 7]));
            }
            else
            {
#pragma unroll
                for(int i = 0; i < 128; ++i)
                    if(ccol0 + i < prm.N)
                        dst[i] = __float2bfloat16_rn(acc[i]);
            }
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    cluster_sync_all();
    if(warp == 1)
    {
        tc_fence_after_sync();
        tmem_dealloc_2cta(tmem_base, 512);
    }
}

} // namespace b200
