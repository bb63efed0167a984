// FP8 x FP8 GEMM with fp32 scales per 128-wide K block: x_scale[M][K/128] (one per activation row and K
// block) and w_scale[N/128][K/128] (one per 128x128 weight block), bf16 output.
//
//   out[m][n] = sum_kb  xs[m][kb] * ws[n/128][kb] * sum_{k in block kb} A[m][k] * B[n][k]
//
// fp32 scales cannot ride the block-scaled MMA (its scales are powers of two), so every K block is
// multiplied unscaled (tcgen05.mma kind::f8f6f4, 4 instructions of K = 32) into one of four TMEM partial
// accumulators, and the 128 epilogue threads (one output row each) promote the finished partial into fp32
// register accumulators with the two scales applied, while the tensor core fills the other partial.
//
// One 128x128 output tile per CTA.  Warps (256 threads): 0 and 7 TMA producers (activations / weights), 1 and 6 MMA
// issuers (even / odd K blocks; 1 owns TMEM), 2..5 promotion + store.  Every barrier wait is bounded (see bounded_wait).
#pragma once
#include "gemm_common.cuh"

namespace b200 {

constexpr int kBlockScaleThreads = 256;
constexpr int kFewRowsThreads    = 256; // + a second MMA issuer warp and a second producer warp
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
    void* out;               // bf16 / fp16 / fp32 [M][N]
    long long ldo;
    int out_mode;            // OutMode (OUT_BF16, OUT_F16 or OUT_F32)
    unsigned int* status;
    // K split of the single-CTA kernel (gridDim.z slices): fp32 partial tiles + one ticket per output tile
    int splits;
    float* ws_partial;
    unsigned int* ws_counter;
    int scales_e8m0;         // few-rows kernel: both scale tensors hold e8m0 bytes (2^(e-127)) instead of floats
    int tma_out;             // few-rows kernel: columns per warp-wide TMA tile store of the output (0: plain stores)
    int cluster;             // few-rows kernel: the slices are the CTAs of one cluster and meet in shared memory
    int pairs_m, tiles_n;    // pair kernel (persistent): 256-row tiles x 256-column tiles of the output
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

// e8m0 byte -> float: 2^(e - 127); 0 is the denormal 2^-127, 255 is NaN
__device__ __forceinline__ float e8m0_to_float(uint32_t e)
{
    return __uint_as_float(e == 0u ? 0x00400000u : (e == 255u ? 0x7FC00000u : e << 23));
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
    auto part_empty_bar = [&](int b) { return bar_base + 192u + 8u * b; };
    constexpr int NP = 4; // TMEM partials (4 x 128 columns: the whole TMEM)
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + kStageBytes * S + 160);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + kStageBytes * S + 164);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kTileP;
    const int col0 = blockIdx.y * kBsTileN;
    // this CTA's K blocks: slice blockIdx.z of prm.splits (all of them without a split)
    const int kb0  = static_cast<int>(static_cast<long long>(prm.k_blocks) * blockIdx.z / prm.splits);
    const int KB   = static_cast<int>(static_cast<long long>(prm.k_blocks) * (blockIdx.z + 1) / prm.splits) - kb0;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            mbar_init(full_bar(s), 2); // one expect_tx arrival per producer warp
            mbar_init(empty_bar(s), 1);
        }
        for(int b = 0; b < NP; ++b)
        {
            mbar_init(part_full_bar(b), 1);
            mbar_init(part_empty_bar(b), 4);
        }
        mbar_init(bar_base + 176u, 4);
        *abort_f = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if(warp == 1)
    {
        tmem_alloc(smem_u32(tmem_ptr_smem), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    // programmatic dependent launch: the set-up above may overlap the previous kernel's tail; nothing below touches
    // global memory before that kernel has completed
    grid_dependency_wait();
    grid_launch_dependents();

    if(warp == 0 || warp == 7)
    {
        // two producer threads: warp 0 loads the activation tiles, warp 7 the weight tiles
        if(lane == 0)
        {
            const bool is_a = (warp == 0);
            // single-thread loops pay every instruction's latency: ring counters, no division
            int issued = 0;
            int s = 0;
            uint32_t phase = 0;
            for(int j = 0; j < KB; ++j)
            {
                if(j >= S && !bounded_wait(empty_bar(s), phase ^ 1u, abort_f, prm.status, ST_TIMEOUT_PRODUCER, j))
                    break;
                const uint32_t stage = smem_base + s * kStageBytes;
                mbar_arrive_expect_tx(full_bar(s), kStageBytes / 2);
                if(is_a)
                    issue_operand_load(prm.a_mode, stage, &map_a, full_bar(s), row0, kb0 + j);
                else
                    issue_operand_load(prm.b_mode, stage + kTileP * kTileKBytes, &map_b, full_bar(s), col0, kb0 + j);
                issued = j + 1;
                if(++s == S)
                {
                    s = 0;
                    phase ^= 1u;
                }
            }
            if(*abort_f)
                for(int j = issued - 1; j >= 0 && j >= issued - S; --j)
                {
                    const uint64_t t0 = global_timer_ns();
                    while(!mbar_try_wait(full_bar(j % S), (j / S) & 1) && global_timer_ns() - t0 < c_wait_ctl.limit_ns) {}
                }
        }
    }
    else if(warp == 1 || warp == 6)
    {
        // two MMA issuers, even K blocks from warp 1 and odd ones from warp 6 (issuing a block costs a single thread
        // about twice as long as the tensor pipe needs for it; the partials of consecutive blocks are independent)
        if(lane == 0)
        {
            const int first = (warp == 1) ? 0 : 1;
            const uint32_t idesc = idesc_f8f6f4_e4m3(kTileP, kBsTileN);
            const bool a_tiled = (prm.a_mode == OPM_TILE16), b_tiled = (prm.b_mode == OPM_TILE16);
            const uint32_t a_lbo = a_tiled ? kTileP * 16u : 16u, a_sbo = a_tiled ? 128u : 1024u, a_lay = a_tiled ? 0u : 2u;
            const uint32_t a_adv = a_tiled ? 2u * kTileP * 16u : 32u;
            const uint32_t b_lbo = b_tiled ? kBsTileN * 16u : 16u, b_sbo = b_tiled ? 128u : 1024u, b_lay = b_tiled ? 0u : 2u;
            const uint32_t b_adv = b_tiled ? 2u * kBsTileN * 16u : 32u;
            // descriptor words once; per MMA only an add on the address field
            const uint32_t a_hi  = static_cast<uint32_t>(make_smem_desc(0, a_lbo, a_sbo, a_lay) >> 32);
            const uint32_t b_hi  = static_cast<uint32_t>(make_smem_desc(0, b_lbo, b_sbo, b_lay) >> 32);
            const uint32_t a_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base, a_lbo, a_sbo, a_lay));
            const uint32_t b_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base + kTileP * kTileKBytes, b_lbo, b_sbo, b_lay));
            const uint32_t a_step = a_adv >> 4, b_step = b_adv >> 4;
            bool ok = true;
            int s = first % S;
            uint32_t phase = (first / S) & 1u;
            for(int j = first; j < KB && ok; j += 2)
            {
                const int b = j & (NP - 1);
                if(j >= NP) // every partial starts free
                    ok = bounded_wait(part_empty_bar(b), ((j / NP) & 1) ^ 1, abort_f, prm.status, ST_TIMEOUT_MMA_SF, j);
                if(ok)
                    ok = bounded_wait(full_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, j);
                if(!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t a_lo = a_lo0 + s * (kStageBytes >> 4), b_lo = b_lo0 + s * (kStageBytes >> 4);
#pragma unroll
                for(int k = 0; k < 4; ++k)
                    mma_f8f6f4(tmem_base + b * kBsTileN, pack_u64(a_lo + k * a_step, a_hi), pack_u64(b_lo + k * b_step, b_hi), idesc,
                               k > 0 ? 1u : 0u);
                tc_commit(empty_bar(s));
                tc_commit(part_full_bar(b));
                if((s += 2) >= S)
                {
                    s -= S;
                    phase ^= 1u;
                }
            }
        }
    }
    else if(warp < 6)
    {
        // promotion + store: thread = output row
        const int quarter    = warp & 3;
        const int r_local    = quarter * 32 + lane;
        const int row        = row0 + r_local;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const bool row_ok    = row < prm.M;
        const float* xs      = prm.x_scale + static_cast<long long>(row_ok ? row : 0) * prm.xs_stride_m + static_cast<long long>(kb0) * prm.xs_stride_k;
        const float* ws      = prm.w_scale + static_cast<long long>(blockIdx.y) * prm.k_blocks + kb0;
        float acc[kBsTileN];
#pragma unroll
        for(int i = 0; i < kBsTileN; ++i)
            acc[i] = 0.f;
        bool ok = true;
        // One K block: wait for its partial, fold it into the accumulators, hand the partial back.
        auto promote = [&](int j, float scale) {
            const int b = j & (NP - 1);
            ok = bounded_wait(part_full_bar(b), (j / NP) & 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, j);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                return;
            tc_fence_after_sync();
            // sixteen columns at a time through two register buffers: the load of the next chunk is in flight while this
            // one is folded in
            uint32_t ra[16], rb[16];
            const uint32_t t0 = tlane + b * kBsTileN;
            tmem_ld_x16_at(t0, ra);
            tmem_ld_wait();
#pragma unroll
            for(int c = 0; c < kBsTileN / 16; ++c)
            {
                if(c + 1 < kBsTileN / 16)
                    tmem_ld_x16_at(t0 + (c + 1) * 16, (c & 1) ? ra : rb);
#pragma unroll
                for(int i = 0; i < 16; ++i)
                    acc[c * 16 + i] = fmaf(__uint_as_float(((c & 1) ? rb : ra)[i]), scale, acc[c * 16 + i]);
                if(c + 1 < kBsTileN / 16)
                    tmem_ld_wait();
            }
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
                mbar_arrive(part_empty_bar(b));
        };
        // The scales of K blocks j and j + 1 wait in registers as loaded (the product is taken when block j's partial is
        // there): a K-block-major x_scale puts every K block on a cache line of its own, an L2 round trip that a
        // look-ahead of one K block does not cover.
        auto ld_x = [&](int j) { return j < KB ? __ldg(xs + static_cast<long long>(j) * prm.xs_stride_k) : 0.f; };
        auto ld_w = [&](int j) { return j < KB ? __ldg(ws + j) : 0.f; };
        float xa = ld_x(0), wa = ld_w(0), xb = ld_x(1), wb = ld_w(1);
        for(int j = 0; j < KB && ok; j += 2)
        {
            const float sa = xa * wa;
            xa = ld_x(j + 2);
            wa = ld_w(j + 2);
            promote(j, sa);
            if(j + 1 < KB && ok)
            {
                const float sb = xb * wb;
                xb = ld_x(j + 3);
                wb = ld_w(j + 3);
                promote(j + 1, sb);
            }
        }
        if(ok && prm.splits > 1)
        {
            // K split: park this slice's tile ([column][row] floats, coalesced), take a ticket; the last slice to arrive
            // adds the slices up in a fixed order (deterministic) and stores the tile
            const unsigned int tile = blockIdx.x * gridDim.y + blockIdx.y;
            float* mine = prm.ws_partial + (static_cast<size_t>(tile) * prm.splits + blockIdx.z) * (kBsTileN * kTileP);
#pragma unroll
            for(int i = 0; i < kBsTileN; ++i)
                mine[i * kTileP + r_local] = acc[i];
            __threadfence();
            // rendezvous of the four promotion warps on an mbarrier (bounded like every other wait here)
            const uint32_t epi_bar = bar_base + 176u;
            unsigned int* ticket   = reinterpret_cast<unsigned int*>(smem_gen + kStageBytes * S + 168);
            __syncwarp();
            if(lane == 0)
                mbar_arrive(epi_bar);
            bool all = bounded_wait(epi_bar, 0, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x1000);
            all      = __all_sync(0xffffffffu, all);
            if(all)
            {
                if(threadIdx.x == 64)
                {
                    *reinterpret_cast<volatile unsigned int*>(ticket) = atomicAdd(prm.ws_counter + tile, 1u);
                    __threadfence_block();
                }
                __syncwarp();
                if(lane == 0)
                    mbar_arrive(epi_bar);
                all = bounded_wait(epi_bar, 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x2000);
                all = __all_sync(0xffffffffu, all);
            }
            ok = all && (*reinterpret_cast<volatile unsigned int*>(ticket) == static_cast<unsigned int>(prm.splits - 1));
            if(ok)
            {
                __threadfence();
                const float* part = prm.ws_partial + static_cast<size_t>(tile) * prm.splits * (kBsTileN * kTileP);
#pragma unroll
                for(int i = 0; i < kBsTileN; ++i)
                    acc[i] = 0.f;
                for(int z = 0; z < prm.splits; ++z)
                {
                    const float* src = part + static_cast<size_t>(z) * (kBsTileN * kTileP);
#pragma unroll
                    for(int i = 0; i < kBsTileN; ++i)
                        acc[i] += __ldcg(src + i * kTileP + r_local);
                }
                if(threadIdx.x == 64)
                    prm.ws_counter[tile] = 0; // ready for the next launch
            }
        }
        if(ok && row_ok)
        {
            const bool vec_ok = ((prm.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(prm.out) & 15) == 0);
            store_row<kBsTileN>(prm.out, prm.out_mode, static_cast<size_t>(row) * prm.ldo + col0, acc, prm.N - col0, vec_ok);
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    if(warp == 1)
    {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}


// ---------------------------------------------------------------------------------------------------------
// Few activation rows (M <= 64): the operands trade places.  128 weight rows are the M side of the MMA and the
// XR (16/32/64) activation rows its N side, so a K block costs 16 KB + XR * 128 B of staging instead of 32 KB,
// the TMEM partial is XR columns wide and a promotion thread (= one output COLUMN n) folds XR values per K block
// with x_scale[m][kb] * w_scale[n/128][kb]; 8 TMEM partials are in flight, so the round trip
// MMA -> commit -> promotion -> release is paid once per 8 K blocks, not per 2.  gridDim.z slices of K meet either
// in shared memory (the slices form one thread-block cluster; every CTA reduces its share of the tile's columns
// and receives the other slices' partial sums of them by st.async) or in the fp32 workspace like in the kernel above.  Warps (256 threads): 0 and 7 TMA producers (weights / activations), 1 and 6 MMA issuers (1 owns TMEM), 2..5 promotion + store.
template <int XR>
__global__ void __launch_bounds__(kFewRowsThreads, 1)
gemm_a8w8_blockscale_fewrows_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                    const __grid_constant__ CUtensorMap map_o, const BlockScaleParams prm)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const int S              = prm.stages;
    constexpr uint32_t kWBytes     = kBsTileN * kTileKBytes;         // 16 KB of weights
    constexpr uint32_t kStageBytes = kWBytes + XR * kTileKBytes;     // + the activation rows
    constexpr int NP               = 8;                              // TMEM partials in flight
    static_assert(XR == 16 || XR == 32 || XR == 64, "activation rows per tile");
    constexpr uint32_t kTmemCols   = NP * XR;
    constexpr uint32_t kSliceBytes = kBsTileN * XR * 4u;             // one CTA's fp32 tile
    // stages | the other slices' tiles (cluster split: written by those CTAs) | barriers and flags
    const uint32_t red_off   = kStageBytes * S;
    // cluster split: every CTA reduces kBsTileN / splits of the tile's columns and receives the other slices' values of them
    const uint32_t red_bytes = prm.cluster ? static_cast<uint32_t>(prm.splits - 1) * (kSliceBytes / static_cast<uint32_t>(prm.splits)) : 0u;
    const uint32_t bar_off   = red_off + red_bytes;
    const uint32_t bar_base  = smem_base + bar_off;
    auto full_bar       = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar      = [&](int s) { return bar_base + 64u + 8u * s; };
    auto part_full_bar  = [&](int b) { return bar_base + 128u + 8u * b; };
    auto part_empty_bar = [&](int b) { return bar_base + 192u + 8u * b; };
    const uint32_t epi_bar     = bar_base + 256u;
    const uint32_t red_bar     = bar_base + 264u;
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + bar_off + 272);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + bar_off + 276);
    unsigned int* ticket       = reinterpret_cast<unsigned int*>(smem_gen + bar_off + 280);
    float* sc_tab              = reinterpret_cast<float*>(smem_gen + bar_off + 512); // [K block of this slice][XR] scale products
    const uint32_t zrank       = prm.cluster ? cluster_ctarank() : blockIdx.z; // K slice
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col0 = blockIdx.x * kBsTileN;
    const int m0   = static_cast<int>(blockIdx.y) * XR; // this CTA's activation rows (more than one tile of rows only for XR = 64)
    const int kb0  = static_cast<int>(static_cast<long long>(prm.k_blocks) * zrank / prm.splits);
    const int KB   = static_cast<int>(static_cast<long long>(prm.k_blocks) * (zrank + 1) / prm.splits) - kb0;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            mbar_init(full_bar(s), 2); // one expect_tx arrival per producer warp
            mbar_init(empty_bar(s), 1);
        }
        for(int b = 0; b < NP; ++b)
        {
            mbar_init(part_full_bar(b), 1);
            mbar_init(part_empty_bar(b), 4);
        }
        mbar_init(epi_bar, 4);
        mbar_init(red_bar, 1);
        *abort_f = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if(warp == 1)
    {
        tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    if(prm.cluster)
        cluster_arrive_release(); // "my barriers exist": checked by the promotion warps before their first remote access
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    // programmatic dependent launch: the set-up above may overlap the previous kernel's tail; nothing below touches
    // global memory before that kernel has completed, and the next kernel's set-up may start from here on
    grid_dependency_wait();
    grid_launch_dependents();

    if(warp == 0 || warp == 7)
    {
        // two producer threads: warp 0 loads the weight tiles, warp 7 the activation rows (a producer needs several
        // hundred cycles per K block at a single thread's instruction latency)
        if(lane == 0)
        {
            const bool is_w = (warp == 0);
            // single-thread loops pay every instruction's latency: ring counters, no division
            int issued = 0;
            int s = 0;
            uint32_t phase = 0;
            for(int j = 0; j < KB; ++j)
            {
                if(j >= S && !bounded_wait(empty_bar(s), phase ^ 1u, abort_f, prm.status, ST_TIMEOUT_PRODUCER, j))
                    break;
                const uint32_t stage = smem_base + s * kStageBytes;
                if(is_w)
                {
                    mbar_arrive_expect_tx(full_bar(s), kWBytes);
                    issue_operand_load(prm.b_mode, stage, &map_b, full_bar(s), col0, kb0 + j);
                }
                else
                {
                    mbar_arrive_expect_tx(full_bar(s), XR * kTileKBytes);
                    issue_operand_load(prm.a_mode, stage + kWBytes, &map_a, full_bar(s), m0, kb0 + j);
                }
                issued = j + 1;
                if(++s == S)
                {
                    s = 0;
                    phase ^= 1u;
                }
            }
            if(*abort_f)
                for(int j = issued - 1; j >= 0 && j >= issued - S; --j)
                {
                    const uint64_t t0 = global_timer_ns();
                    while(!mbar_try_wait(full_bar(j % S), (j / S) & 1) && global_timer_ns() - t0 < c_wait_ctl.limit_ns) {}
                }
        }
    }
    else if(warp == 1 || warp == 6)
    {
        // two MMA issuers, even K blocks from warp 1 and odd ones from warp 6: an issuer needs ~600 cycles per K block
        // (a barrier wait, four MMAs and two commits at a single thread's instruction latency), the tensor pipe far
        // less, and the partials of consecutive K blocks are independent
        if(lane == 0)
        {
            const int first = (warp == 1) ? 0 : 1;
            const uint32_t idesc = idesc_f8f6f4_e4m3(kBsTileN, XR);
            const bool w_tiled = (prm.b_mode == OPM_TILE16), x_tiled = (prm.a_mode == OPM_TILE16);
            const uint32_t w_lbo = w_tiled ? kBsTileN * 16u : 16u, w_sbo = w_tiled ? 128u : 1024u, w_lay = w_tiled ? 0u : 2u;
            const uint32_t w_adv = w_tiled ? 2u * kBsTileN * 16u : 32u;
            const uint32_t x_lbo = x_tiled ? XR * 16u : 16u, x_sbo = x_tiled ? 128u : 1024u, x_lay = x_tiled ? 0u : 2u;
            const uint32_t x_adv = x_tiled ? 2u * XR * 16u : 32u;
            // descriptor words once; per MMA only an add on the address field (this thread pays every instruction's
            // latency, so no division, no descriptor assembly and no wait that cannot block inside the loop)
            const uint32_t w_hi  = static_cast<uint32_t>(make_smem_desc(0, w_lbo, w_sbo, w_lay) >> 32);
            const uint32_t x_hi  = static_cast<uint32_t>(make_smem_desc(0, x_lbo, x_sbo, x_lay) >> 32);
            const uint32_t w_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base, w_lbo, w_sbo, w_lay));
            const uint32_t x_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base + kWBytes, x_lbo, x_sbo, x_lay));
            const uint32_t w_step = w_adv >> 4, x_step = x_adv >> 4;
            bool ok = true;
            int s = first % S, b = first;
            uint32_t phase = (first / S) & 1u, bphase = 0;
            for(int j = first; j < KB && ok; j += 2)
            {
                if(j >= NP) // the first NP partials are free
                    ok = bounded_wait(part_empty_bar(b), bphase ^ 1u, abort_f, prm.status, ST_TIMEOUT_MMA_SF, j);
                if(ok)
                    ok = bounded_wait(full_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, j);
                if(!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t w_lo = w_lo0 + s * (kStageBytes >> 4), x_lo = x_lo0 + s * (kStageBytes >> 4);
#pragma unroll
                for(int k = 0; k < 4; ++k)
                    mma_f8f6f4(tmem_base + b * XR, pack_u64(w_lo + k * w_step, w_hi), pack_u64(x_lo + k * x_step, x_hi), idesc,
                               k > 0 ? 1u : 0u);
                tc_commit(empty_bar(s));
                tc_commit(part_full_bar(b));
                if((s += 2) >= S)
                {
                    s -= S;
                    phase ^= 1u;
                }
                if((b += 2) >= NP) // (the odd issuer passes NP + 1)
                {
                    b -= NP;
                    bphase ^= 1u;
                }
            }
        }
    }
    else if(warp < 6)
    {
        // promotion + store: thread = output column n, TMEM columns = output rows m
        const int quarter    = warp & 3;
        const int r_local    = quarter * 32 + lane;
        const int n          = col0 + r_local;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        float acc[XR];
#pragma unroll
        for(int i = 0; i < XR; ++i)
            acc[i] = 0.f;
        bool ok = true;
        if(prm.cluster && threadIdx.x == 64)
            mbar_arrive_expect_tx(red_bar, red_bytes);
        // x_scale[m][kb] * w_scale[n/128][kb] of this slice goes to shared memory once (while the first loads are in
        // flight); the K loop then reads four products per broadcast load instead of assembling XR global addresses
        // per K block, which a warp that has its scheduler to itself pays instruction by instruction
        for(int it = threadIdx.x - 64; it < KB * XR; it += 128)
        {
            const int j = it / XR, i = it - j * XR;
            const long long xo = static_cast<long long>(m0 + i < prm.M ? m0 + i : 0) * prm.xs_stride_m + static_cast<long long>(kb0 + j) * prm.xs_stride_k;
            const long long wo = static_cast<long long>(blockIdx.x) * prm.k_blocks + kb0 + j;
            sc_tab[it] = prm.scales_e8m0
                             ? e8m0_to_float(__ldg(reinterpret_cast<const uint8_t*>(prm.x_scale) + xo)) *
                                   e8m0_to_float(__ldg(reinterpret_cast<const uint8_t*>(prm.w_scale) + wo))
                             : __ldg(prm.x_scale + xo) * __ldg(prm.w_scale + wo);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory"); // the four promotion warps (all of them always get here)
        for(int j = 0; j < KB && ok; ++j)
        {
            const int b = j % NP;
            float sc[XR];
#pragma unroll
            for(int i = 0; i < XR; i += 4)
            {
                const float4 t = *reinterpret_cast<const float4*>(sc_tab + j * XR + i);
                sc[i] = t.x;
                sc[i + 1] = t.y;
                sc[i + 2] = t.z;
                sc[i + 3] = t.w;
            }
            ok = bounded_wait(part_full_bar(b), (j / NP) & 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, j);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                break;
            tc_fence_after_sync();
            uint32_t r[XR];
#pragma unroll
            for(int c = 0; c < XR / 16; ++c)
                tmem_ld_x16_at(tlane + b * XR + c * 16, r + c * 16);
            tmem_ld_wait();
#pragma unroll
            for(int i = 0; i < XR; ++i)
                acc[i] = fmaf(__uint_as_float(r[i]), sc[i], acc[i]);
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
                mbar_arrive(part_empty_bar(b));
        }
        bool owns = true; // this thread stores its output column
        if(prm.cluster)
            cluster_wait_acquire(); // every CTA of the cluster has initialised its barriers (they all ran a K loop since)
        if(ok && prm.cluster)
        {
            // Cluster split, reduce-scatter: CTA z adds up columns [z * per, (z + 1) * per) of the tile (per = 128 /
            // splits).  A thread whose column belongs to another CTA sends its XR partial sums to that CTA's shared
            // memory ([source slice][column][m] floats; the bytes are counted on that CTA's barrier, nothing is waited
            // for); a thread that owns its column waits for the other slices' values, adds them in rank order and stores.
            const uint32_t per   = static_cast<uint32_t>(kBsTileN) / static_cast<uint32_t>(prm.splits);
            const uint32_t owner = static_cast<uint32_t>(r_local) / per;
            const uint32_t col   = static_cast<uint32_t>(r_local) - owner * per;
            owns                 = (owner == zrank);
            if(!owns)
            {
                const uint32_t slot    = zrank < owner ? zrank : zrank - 1u; // this slice's place among the owner's sources
                const uint32_t dst     = map_to_cta(smem_base + red_off, owner) + (slot * per + col) * (XR * 4u);
                const uint32_t dst_bar = map_to_cta(red_bar, owner);
#pragma unroll
                for(int i = 0; i < XR; i += 4)
                    st_async_v4(dst + i * 4u, __float_as_uint(acc[i]), __float_as_uint(acc[i + 1]), __float_as_uint(acc[i + 2]),
                                __float_as_uint(acc[i + 3]), dst_bar);
            }
            if(__any_sync(0xffffffffu, owns)) // (a warp may hold columns of two owners when per < 32)
            {
                ok = bounded_wait(red_bar, 0, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x3000);
                ok = __all_sync(0xffffffffu, ok);
                if(ok && owns)
                {
                    const float4* red = reinterpret_cast<const float4*>(smem_gen + red_off);
                    for(uint32_t z = 0; z + 1 < static_cast<uint32_t>(prm.splits); ++z)
                    {
                        const float4* src = red + static_cast<size_t>(z * per + col) * (XR / 4);
#pragma unroll
                        for(int i = 0; i < XR; i += 4)
                        {
                            const float4 t = src[i / 4];
                            acc[i] += t.x;
                            acc[i + 1] += t.y;
                            acc[i + 2] += t.z;
                            acc[i + 3] += t.w;
                        }
                    }
                }
            }
        }
        else if(ok && prm.splits > 1)
        {
            // K split: park this slice ([m][n] floats), take a ticket; the last slice to arrive adds them in a fixed order
            const unsigned int tile = blockIdx.y * gridDim.x + blockIdx.x;
            float* mine = prm.ws_partial + (static_cast<size_t>(tile) * prm.splits + blockIdx.z) * (XR * kBsTileN);
#pragma unroll
            for(int i = 0; i < XR; ++i)
                if(m0 + i < prm.M)
                    mine[i * kBsTileN + r_local] = acc[i];
            __threadfence();
            __syncwarp();
            if(lane == 0)
                mbar_arrive(epi_bar);
            bool all = bounded_wait(epi_bar, 0, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x1000);
            all      = __all_sync(0xffffffffu, all);
            if(all)
            {
                if(threadIdx.x == 64)
                {
                    *reinterpret_cast<volatile unsigned int*>(ticket) = atomicAdd(prm.ws_counter + tile, 1u);
                    __threadfence_block();
                }
                __syncwarp();
                if(lane == 0)
                    mbar_arrive(epi_bar);
                all = bounded_wait(epi_bar, 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x2000);
                all = __all_sync(0xffffffffu, all);
            }
            ok = all && (*reinterpret_cast<volatile unsigned int*>(ticket) == static_cast<unsigned int>(prm.splits - 1));
            if(ok)
            {
                __threadfence();
                const float* part = prm.ws_partial + static_cast<size_t>(tile) * prm.splits * (XR * kBsTileN);
#pragma unroll
                for(int i = 0; i < XR; ++i)
                    acc[i] = 0.f;
                for(int z = 0; z < prm.splits; ++z)
                {
                    const float* src = part + static_cast<size_t>(z) * (XR * kBsTileN);
#pragma unroll
                    for(int i = 0; i < XR; ++i)
                        if(m0 + i < prm.M)
                            acc[i] += __ldcg(src + i * kBsTileN + r_local);
                }
                if(threadIdx.x == 64)
                    prm.ws_counter[tile] = 0; // ready for the next launch
            }
        }
        if(prm.tma_out)
        {
            // Every warp stages the columns it owns ([m][column] bf16, prm.tma_out of them per row: 32, or 16 when the
            // cluster split leaves a CTA half a warp's columns) in a retired operand stage and stores them as one TMA
            // tile, which clips rows >= M and columns >= N; cheaper at the end of a short kernel than XR scattered
            // 2-byte stores per thread.
            const uint32_t mask = __ballot_sync(0xffffffffu, ok && owns);
            if(mask != 0u)
            {
                const int lead   = __ffs(mask) - 1;              // first owning lane of this warp
                const int wcols  = prm.tma_out;
                uint8_t* stg     = smem_gen + (warp - 2) * (XR * 64);
                uint16_t* t      = reinterpret_cast<uint16_t*>(stg);
                if(ok && owns)
                {
#pragma unroll
                    for(int i = 0; i < XR; ++i)
                        t[i * wcols + (lane - lead)] = cvt_out16(acc[i], prm.out_mode == OUT_F16);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if(lane == lead && n < prm.N) // (a tile that starts inside the output; what sticks out is clipped)
                {
                    tma_store_2d(&map_o, smem_base + (warp - 2) * (XR * 64), (n) * 2, m0);
                    bulk_commit_group();
                    bulk_wait_group_read<0>(); // the store has read its source before the CTA retires (see gemm_persistent.cuh)
                }
            }
        }
        else if(ok && owns && n < prm.N)
        {
#pragma unroll
            for(int i = 0; i < XR; ++i)
                if(m0 + i < prm.M)
                    store_out(prm.out, static_cast<size_t>(m0 + i) * prm.ldo + n, acc[i], prm.out_mode);
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    // no cluster rendezvous at the end: the only remote traffic into a CTA are the partial sums of the columns it owns,
    // and the warp that owns them has waited for every byte (red barrier) before the CTA gets here
    if(warp == 1)
    {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}


// ---------------------------------------------------------------------------------------------------------
// Same arithmetic on CTA pairs: 256 x 256 output tiles (cta_group::2), a persistent pair walking a static list of
// them, so that barrier set-up, TMEM allocation and the pipeline fill are paid once and a tile's rows go out while the
// next tile's operands arrive and its first K blocks are multiplied.  Every CTA stages its own 128 rows of A and its
// own 128 of the tile's 256 rows of B per K block (half the operand bytes per flop of the 128 x 128 tile), the leader
// issues 256 x 256 x 32 MMAs into one of two 256-column TMEM partials, and eight promotion warps per CTA (two per
// TMEM lane quarter, 128 columns each) fold the finished partial into fp32 registers with
// x_scale[m][kb] * w_scale[n/128][kb]: 16 columns per tcgen05.ld through two register buffers, the scales loaded two
// K blocks ahead.  16-bit outputs leave as TMA tile stores from a staging buffer per warp, others as plain stores.
// Warps (352 threads): 0 TMA producer, 1 MMA issuer (leader) + TMEM owner, 2..9 promotion + store, 10 descriptor prefetch.
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
                                 const __grid_constant__ CUtensorMap map_o, const BlockScaleParams prm)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const int S              = prm.stages;
    constexpr uint32_t kStageBytes = 2u * kTileP * kTileKBytes; // 16 KB of A + 16 KB of B per CTA
    // stages | one 4 KB output staging buffer per promotion warp (32 rows x 64 columns of 16 bits, 128-byte swizzle) | barriers
    constexpr uint32_t kEpiBytes = 8u * 4096u;
    const uint32_t epi_off   = kStageBytes * S;
    const uint32_t bar_base  = smem_base + epi_off + kEpiBytes;
    auto full_bar       = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar      = [&](int s) { return bar_base + 64u + 8u * s; };
    auto part_full_bar  = [&](int b) { return bar_base + 128u + 8u * b; };
    auto part_empty_bar = [&](int b) { return bar_base + 144u + 8u * b; };
    const uint32_t drain_bar   = bar_base + 160u;
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + epi_off + kEpiBytes + 168);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + epi_off + kEpiBytes + 172);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_ctarank();
    const bool leader    = (crank == 0);
    const int KB         = prm.k_blocks;
    // persistent: cluster c takes tiles c, c + clusters, ...; consecutive tiles share a column tile of B (L2)
    const int n_clusters = static_cast<int>(gridDim.x >> 1);
    const int tile0      = static_cast<int>(blockIdx.x >> 1);
    const int n_tiles    = prm.pairs_m * prm.tiles_n;
    auto tile_row0 = [&](int t) { return ((t % prm.pairs_m) * 2 + static_cast<int>(crank)) * kTileP; };
    auto tile_col0 = [&](int t) { return (t / prm.pairs_m) * kBsPairN; };

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
        if(prm.tma_out)
            tma_prefetch_desc(&map_o);
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
    // programmatic dependent launch (see the 128 x 128 kernel)
    grid_dependency_wait();
    grid_launch_dependents();

    if(warp == 0)
    {
        if(lane == 0)
        {
            const uint32_t full0 = map_to_cta(full_bar(0), 0);
            int s = 0;
            uint32_t phase = 0;
            bool live = true;
            for(int t = tile0; t < n_tiles && live; t += n_clusters)
            {
            const int row0 = tile_row0(t), col0 = tile_col0(t);
            for(int j = 0; j < KB; ++j)
            {
                if(!bounded_wait(empty_bar(s), phase ^ 1u, abort_f, prm.status, ST_TIMEOUT_PRODUCER, j))
                {
                    live = false;
                    break;
                }
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
            uint32_t g = 0; // K blocks issued so far, over all tiles: partial g & 1, its barriers' phase (g >> 1) & 1
            for(int t = tile0; t < n_tiles && ok; t += n_clusters)
            for(int j = 0; j < KB && ok; ++j, ++g)
            {
                const int b = static_cast<int>(g & 1u);
                ok = bounded_wait(part_empty_bar(b), ((g >> 1) & 1u) ^ 1u, abort_f, prm.status, ST_TIMEOUT_MMA_SF, j);
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
                while(!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < c_wait_ctl.limit_ns) {}
            }
        }
    }
    else if(warp < 10)
    {
        // promotion + store: thread = output row, 128 of the tile's 256 columns
        const int quarter    = warp & 3;
        const int half       = (warp - 2) >> 2;
        const int r_local    = quarter * 32 + lane;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 128;
        const uint32_t part_empty_leader = map_to_cta(part_empty_bar(0), 0);
        const bool vec_ok    = ((prm.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(prm.out) & 15) == 0);
        bool ok = true;
        uint32_t g = 0;
        for(int t = tile0; t < n_tiles && ok; t += n_clusters)
        {
            const int row        = tile_row0(t) + r_local;
            const int ccol0      = tile_col0(t) + half * 128;
            const bool row_ok    = row < prm.M;
            const float* xs      = prm.x_scale + static_cast<long long>(row_ok ? row : 0) * prm.xs_stride_m;
            const int nblk       = min(ccol0 / 128, (prm.N + 127) / 128 - 1);
            const float* ws      = prm.w_scale + static_cast<long long>(nblk) * KB;
            float acc[128];
#pragma unroll
            for(int i = 0; i < 128; ++i)
                acc[i] = 0.f;
            // One K block: wait for its partial, fold it into the accumulators, hand the partial back.
            auto promote = [&](int j, float scale) {
                const int b = static_cast<int>(g & 1u);
                ok = bounded_wait(part_full_bar(b), (g >> 1) & 1u, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, j);
                ok = __all_sync(0xffffffffu, ok);
                if(!ok)
                    return;
                tc_fence_after_sync();
                // sixteen columns at a time through two register buffers: the load of the next chunk is in flight while
                // this one is folded in
                uint32_t ra[16], rb[16];
                const uint32_t t0 = tlane + b * kBsPairN;
                tmem_ld_x16_at(t0, ra);
                tmem_ld_wait();
#pragma unroll
                for(int c = 0; c < 8; ++c)
                {
                    if(c < 7)
                        tmem_ld_x16_at(t0 + (c + 1) * 16, (c & 1) ? ra : rb);
#pragma unroll
                    for(int i = 0; i < 16; ++i)
                        acc[c * 16 + i] = fmaf(__uint_as_float(((c & 1) ? rb : ra)[i]), scale, acc[c * 16 + i]);
                    if(c < 7)
                        tmem_ld_wait();
                }
                tc_fence_before_sync();
                __syncwarp();
                if(lane == 0)
                    mbar_arrive_cluster(part_empty_leader + 8u * b);
                ++g;
            };
            // The scales of K blocks j and j + 1 wait in registers as loaded (the product is taken when block j's partial
            // is there): a K-block-major x_scale puts every K block on a cache line of its own, an L2 round trip that a
            // look-ahead of one K block no longer covers.
            auto ld_x = [&](int j) { return j < KB ? __ldg(xs + static_cast<long long>(j) * prm.xs_stride_k) : 0.f; };
            auto ld_w = [&](int j) { return j < KB ? __ldg(ws + j) : 0.f; };
            float xa = ld_x(0), wa = ld_w(0), xb = ld_x(1), wb = ld_w(1);
            for(int j = 0; j < KB && ok; j += 2)
            {
                const float sa = xa * wa;
                xa = ld_x(j + 2);
                wa = ld_w(j + 2);
                promote(j, sa);
                if(j + 1 < KB && ok)
                {
                    const float sb = xb * wb;
                    xb = ld_x(j + 3);
                    wb = ld_w(j + 3);
                    promote(j + 1, sb);
                }
            }
            // (the tensor core is already at work on the next tile's first K blocks while the rows go out)
            if(ok && prm.tma_out)
            {
                // 16-bit outputs: the warp's 32 rows x 128 columns leave as two tile stores of 64 columns, staged in this
                // warp's buffer with the 128-byte swizzle the store expects; the store clips rows >= M and columns >= N
                const bool f16       = (prm.out_mode == OUT_F16);
                const uint32_t boff  = epi_off + static_cast<uint32_t>(warp - 2) * 4096u;
                uint8_t* rowp        = smem_gen + boff + lane * 128;
                const int warp_row0  = tile_row0(t) + quarter * 32;
#pragma unroll
                for(int c = 0; c < 2; ++c)
                {
                    if(lane == 0)
                        bulk_wait_group_read<0>(); // the store that last used the buffer has read it
                    __syncwarp();
#pragma unroll
                    for(int q = 0; q < 8; ++q)
                        *reinterpret_cast<uint4*>(rowp + ((q ^ (lane & 7)) * 16)) =
                            make_uint4(pack_out16x2(acc[c * 64 + 8 * q], acc[c * 64 + 8 * q + 1], f16),
                                       pack_out16x2(acc[c * 64 + 8 * q + 2], acc[c * 64 + 8 * q + 3], f16),
                                       pack_out16x2(acc[c * 64 + 8 * q + 4], acc[c * 64 + 8 * q + 5], f16),
                                       pack_out16x2(acc[c * 64 + 8 * q + 6], acc[c * 64 + 8 * q + 7], f16));
                    fence_proxy_async_smem();
                    __syncwarp();
                    if(lane == 0 && warp_row0 < prm.M && ccol0 + c * 64 < prm.N)
                    {
                        tma_store_2d(&map_o, smem_base + boff, (ccol0 + c * 64) * 2, warp_row0);
                        bulk_commit_group();
                    }
                }
            }
            else if(ok && row_ok && ccol0 < prm.N)
                store_row<128>(prm.out, prm.out_mode, static_cast<size_t>(row) * prm.ldo + ccol0, acc, prm.N - ccol0, vec_ok);
        }
        if(lane == 0)
            bulk_wait_group_read<0>(); // the last stores have read this warp's buffer before the CTA retires
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

// ---------------------------------------------------------------------------------------------------------
// CTA pairs on a 256 x 128 output tile.  The 256 x 256 tile above keeps 128 fp32 accumulators per promotion thread and
// has registers left for a quarter of a TMEM partial at a time: four loads per K block, each queued behind the MMAs of
// the next K block, and the partial is released only after the last of them.  Here a promotion thread owns 64 columns:
// ONE tcgen05.ld brings its whole share of a partial into registers, the partial goes back to the tensor core at once
// (before the multiply-adds), and with 128-column partials TMEM holds four of them, so the MMAs run up to three K
// blocks ahead.  Per K block every CTA stages 16 KB of A and 8 KB (its 64 of the tile's 128 rows) of B.
// Warps (352 threads): 0 TMA producer, 1 MMA issuer (leader) + TMEM owner, 2..9 promotion + store, 10 descriptor prefetch.
constexpr int kBsPairNarrowN = 128;

__global__ void __launch_bounds__(kBlockScalePairThreads, 1)
gemm_a8w8_blockscale_pair_narrow_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                        const BlockScaleParams prm)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const int S              = prm.stages;
    constexpr uint32_t kABytes     = kTileP * kTileKBytes;               // 16 KB: this CTA's 128 rows of A
    constexpr uint32_t kBRows      = kBsPairNarrowN / 2;                 // this CTA's 64 of the tile's 128 rows of B
    constexpr uint32_t kStageBytes = kABytes + kBRows * kTileKBytes;     // 24 KB
    constexpr int NP               = 4;                                  // TMEM partials of 128 columns
    const uint32_t bar_base  = smem_base + kStageBytes * S;
    auto full_bar       = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar      = [&](int s) { return bar_base + 64u + 8u * s; };
    auto part_full_bar  = [&](int b) { return bar_base + 128u + 8u * b; };
    auto part_empty_bar = [&](int b) { return bar_base + 160u + 8u * b; };
    const uint32_t drain_bar   = bar_base + 192u;
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + kStageBytes * S + 200);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + kStageBytes * S + 204);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_ctarank();
    const bool leader    = (crank == 0);
    const int pair_x     = blockIdx.x >> 1;                 // 256-row tile index
    const int row0       = (pair_x * 2 + static_cast<int>(crank)) * kTileP;
    const int col0       = blockIdx.y * kBsPairNarrowN;
    const int KB         = prm.k_blocks;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            mbar_init(full_bar(s), 2);  // one expect_tx arrival per CTA of the pair
            mbar_init(empty_bar(s), 1);
        }
        for(int b = 0; b < NP; ++b)
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
    // programmatic dependent launch (see the 128 x 128 kernel)
    grid_dependency_wait();
    grid_launch_dependents();

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
                const int brow = col0 + static_cast<int>(crank * kBRows);
                if(prm.b_mode == OPM_ROWMAJOR)
                    tma_load_2d_pair(stage + kABytes, &map_b, bar, j * kTileKBytes, brow);
                else
                    tma_load_3d_pair(stage + kABytes, &map_b, bar, 0, brow >> 4, j * (kTileKBytes / 16));
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
            const uint32_t idesc = idesc_f8f6f4_e4m3(2 * kTileP, kBsPairNarrowN);
            const bool a_tiled = (prm.a_mode == OPM_TILE16), b_tiled = (prm.b_mode == OPM_TILE16);
            const uint32_t a_lbo = a_tiled ? kTileP * 16u : 16u, a_sbo = a_tiled ? 128u : 1024u, a_lay = a_tiled ? 0u : 2u;
            const uint32_t a_step = (a_tiled ? 2u * kTileP * 16u : 32u) >> 4;
            const uint32_t b_lbo = b_tiled ? kBRows * 16u : 16u, b_sbo = b_tiled ? 128u : 1024u, b_lay = b_tiled ? 0u : 2u;
            const uint32_t b_step = (b_tiled ? 2u * kBRows * 16u : 32u) >> 4;
            const uint32_t a_hi  = static_cast<uint32_t>(make_smem_desc(0, a_lbo, a_sbo, a_lay) >> 32);
            const uint32_t b_hi  = static_cast<uint32_t>(make_smem_desc(0, b_lbo, b_sbo, b_lay) >> 32);
            const uint32_t a_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base, a_lbo, a_sbo, a_lay));
            const uint32_t b_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base + kABytes, b_lbo, b_sbo, b_lay));
            bool ok = true;
            int s = 0;
            uint32_t phase = 0;
            for(int j = 0; j < KB && ok; ++j)
            {
                const int b = j & (NP - 1);
                ok = bounded_wait(part_empty_bar(b), ((j >> 2) & 1) ^ 1, abort_f, prm.status, ST_TIMEOUT_MMA_SF, j);
                if(ok)
                    ok = bounded_wait(full_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, j);
                if(!ok)
                    break;
                tc_fence_after_sync();
                const uint32_t a_lo = a_lo0 + s * (kStageBytes >> 4), b_lo = b_lo0 + s * (kStageBytes >> 4);
#pragma unroll
                for(int k = 0; k < 4; ++k)
                    mma_f8f6f4_2cta(tmem_base + b * kBsPairNarrowN, pack_u64(a_lo + k * a_step, a_hi), pack_u64(b_lo + k * b_step, b_hi), idesc,
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
                while(!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < c_wait_ctl.limit_ns) {}
            }
        }
    }
    else if(warp < 10)
    {
        // promotion + store: thread = output row, 64 of the tile's 128 columns
        const int quarter    = warp & 3;
        const int half       = (warp - 2) >> 2;
        const int r_local    = quarter * 32 + lane;
        const int row        = row0 + r_local;
        const int ccol0      = col0 + half * 64;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 64;
        const bool row_ok    = row < prm.M;
        const float* xs      = prm.x_scale + static_cast<long long>(row_ok ? row : 0) * prm.xs_stride_m;
        const float* ws      = prm.w_scale + static_cast<long long>(blockIdx.y) * KB; // the tile is one 128-column scale block wide
        const uint32_t part_empty_leader = map_to_cta(part_empty_bar(0), 0);
        float acc[64];
#pragma unroll
        for(int i = 0; i < 64; ++i)
            acc[i] = 0.f;
        bool ok = true;
        // The scales of the next four K blocks wait in registers: with the shared-memory carve-out at its maximum the L1
        // that is left does not hold a line per row, so every scale load is an L2 round trip, which a look-ahead of
        // one K block does not cover.
        float xq[NP], wq[NP];
#pragma unroll
        for(int d = 0; d < NP; ++d)
        {
            xq[d] = (d < KB) ? __ldg(xs + static_cast<long long>(d) * prm.xs_stride_k) : 0.f;
            wq[d] = (d < KB) ? __ldg(ws + d) : 0.f;
        }
        for(int j0 = 0; j0 < KB && ok; j0 += NP)
        {
#pragma unroll
            for(int d = 0; d < NP; ++d)
            {
                const int j = j0 + d; // partial j & 3 = d
                if(j >= KB || !ok)
                    break;
                const float scale = xq[d] * wq[d];
                if(j + NP < KB)
                {
                    xq[d] = __ldg(xs + static_cast<long long>(j + NP) * prm.xs_stride_k);
                    wq[d] = __ldg(ws + j + NP);
                }
                ok = bounded_wait(part_full_bar(d), (j >> 2) & 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, j);
                ok = __all_sync(0xffffffffu, ok);
                if(!ok)
                    break;
                tc_fence_after_sync();
                uint32_t r[64];
                tmem_ld_x64(tlane + d * kBsPairNarrowN, r);
                tmem_ld_wait();
                // the partial is in registers: hand it back before the arithmetic
                tc_fence_before_sync();
                __syncwarp();
                if(lane == 0)
                    mbar_arrive_cluster(part_empty_leader + 8u * d);
#pragma unroll
                for(int i = 0; i < 64; ++i)
                    acc[i] = fmaf(__uint_as_float(r[i]), scale, acc[i]);
            }
        }
        if(ok && row_ok && ccol0 < prm.N)
        {
            const bool vec_ok = ((prm.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(prm.out) & 15) == 0);
            store_row<64>(prm.out, prm.out_mode, static_cast<size_t>(row) * prm.ldo + ccol0, acc, prm.N - ccol0, vec_ok);
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
