// Warp-specialised tcgen05 GEMM for sm_100a:  D[p][q] = sum_k P[p][k] * Q[q][k]  (both K-major).
//
// "P" is the operand that fills the 128-row M slot of the UMMA instruction and ends up on the
// 128 TMEM lanes; "Q" fills the N slot (BN = 16..256 columns).  The host decides which of
// (activations, weights) plays P and which plays Q: for tall problems P = activations, for
// decode-sized problems P = weights ("swap"), so that the weight matrix is streamed once
// through full-height MMA tiles while the handful of activation rows sit in the N slot.
//
// Operand staging (TMA, never multicast):
//   mode 0  row-major [rows][K bytes]          -> 128-byte-swizzled [rows][128 B] tiles
//   mode 1  16x16-byte tile-major (the layout shuffle_weight(layout=(16,16)) and the
//           16x16 tile transpose produce)       -> un-swizzled [16-B K chunk][rows][16 B]
//           tiles, which is exactly the canonical "interleaved" K-major core-matrix layout,
//           so pre-shuffled weights are consumed as they are, 256 contiguous bytes per request
//   mode 2  (rows/2, K/128, 2, 128) activation tiling -> 128-byte-swizzled tiles
//
// Block scales (UE8M0 per 32 along K) travel GMEM -> SMEM in their wire layout by TMA, are
// re-ordered in shared memory by one warp into the 32x16-byte atoms tcgen05.cp wants, and
// are copied to TMEM by the MMA thread right before the MMAs that use them.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer (+ TMEM owner), warp 2 scale re-order,
// warps 3..6 epilogue (TMEM -> registers -> bf16 -> global, or fp32 split-K partials with a
// last-arriver reduction: no CTA ever waits for another CTA).
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in `status`, raises a
// CTA-wide abort flag, drains its own TMA traffic, frees TMEM and returns.
#pragma once
#include "gemm_common.cuh"

namespace b200 {

struct GemmParams
{
    int rows_p, rows_q;       // valid rows of P and Q
    int num_k_iters;          // ceil(K bytes / 128)
    int kblocks;              // valid 32-element scale blocks along K
    int bn;                   // UMMA N: 16, 32, 64, 128 or 256
    int stages;
    int p_mode, q_mode;       // OperandMode
    int sf_groups_p, sf_groups_q; // 32-row scale groups fetched per tile
    int transposed_out;       // 0: out[p][q], 1: out[q][p]
    int tmem_cols;            // power of two >= 32
    int sf_tmem_base;         // first TMEM column used for scale factors
    __nv_bfloat16* out;
    long long ldo;            // elements
    const void* bias;         // fp32 or bf16, indexed by the weight row; may be null
    int bias_is_bf16;
    int bias_on_q;            // 1: bias index is the q coordinate, 0: the p coordinate
    float alpha, beta;
    float* ws_partial;        // split-K partials (null when gridDim.z == 1)
    unsigned int* ws_counter; // one ticket counter per output tile, zero between launches
    unsigned int* status;     // 4 words
    unsigned long long* trace; // optional 64-slot timestamp record of CTA (0,0,0); null = off
};

struct SmemLayout
{
    uint32_t stage_bytes, q_off, sfp_off, sfq_off, bar_off, total;
};

__host__ __device__ inline SmemLayout make_smem_layout(int kind, int bn, int stages)
{
    SmemLayout L;
    uint32_t q_bytes = static_cast<uint32_t>(bn) * kTileKBytes;
    q_bytes          = (q_bytes + 1023u) & ~1023u;
    L.q_off          = kTileP * kTileKBytes;
    L.sfp_off        = L.q_off + q_bytes;
    L.sfq_off        = L.sfp_off + (kind == KIND_BF16 ? 0u : 1024u);
    L.stage_bytes    = L.sfq_off + (kind == KIND_BF16 ? 0u : 2048u);
    L.bar_off        = L.stage_bytes * static_cast<uint32_t>(stages);
    L.total          = L.bar_off + 512u;
    return L;
}

template <int KIND, int SFW>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                    const __grid_constant__ CUtensorMap map_sfp, const __grid_constant__ CUtensorMap map_sfq,
                    const GemmParams prm)
{
    constexpr bool kScaled   = (KIND != KIND_BF16);
    constexpr int kAtomsK    = (KIND == KIND_MXF4) ? 2 : 1; // 512-byte scale atoms per 128 rows per stage
    constexpr int kSfChunk   = (SFW == SFW_E8M0_SHUFFLE) ? 256 : 128 * kAtomsK; // wire bytes per 32-row group per stage

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const SmemLayout L       = make_smem_layout(KIND, prm.bn, prm.stages);

    const uint32_t bar_base    = smem_base + L.bar_off;
    auto full_bar              = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar             = [&](int s) { return bar_base + 64u + 8u * s; };
    auto sf_bar                = [&](int s) { return bar_base + 128u + 8u * s; };
    const uint32_t accum_bar   = bar_base + 192u;
    const uint32_t drain_bar   = bar_base + 200u;
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + L.bar_off + 208);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + L.bar_off + 212);
    uint32_t* ticket_smem      = reinterpret_cast<uint32_t*>(smem_gen + L.bar_off + 216);
    const uint32_t epi_bar     = bar_base + 224u; // the four epilogue warps meet here (bounded)

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const bool tracing = (prm.trace != nullptr) && (blockIdx.x | blockIdx.y | blockIdx.z) == 0;
    auto stamp = [&](int slot) { if(tracing && slot < 64) prm.trace[slot] = static_cast<unsigned long long>(clock64()); };
    if(threadIdx.x == 0) stamp(0);
    const int bn   = prm.bn;
    const int S    = prm.stages;

    // this CTA's slice of the K loop (host guarantees gridDim.z <= num_k_iters)
    const int splits  = gridDim.z;
    const int it_beg  = static_cast<int>((static_cast<long long>(prm.num_k_iters) * blockIdx.z) / splits);
    const int it_end  = static_cast<int>((static_cast<long long>(prm.num_k_iters) * (blockIdx.z + 1)) / splits);
    const int n_iters = it_end - it_beg;
    const int row_p0  = blockIdx.x * kTileP;
    const int row_q0  = blockIdx.y * bn;

    // A failure recorded by an earlier CTA or launch (and not yet read by the host) ends this CTA at once.
    if(threadIdx.x == 0)
        *ticket_smem = *reinterpret_cast<volatile unsigned int*>(prm.status);
    __syncthreads();
    if(*ticket_smem != 0)
        return;
    __syncthreads();

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(sf_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        mbar_init(drain_bar, 1);
        mbar_init(epi_bar, 4);
        *abort_f = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if(warp == 0 && lane == 0)
    {
        tma_prefetch_desc(&map_p);
        tma_prefetch_desc(&map_q);
        if(kScaled)
        {
            tma_prefetch_desc(&map_sfp);
            tma_prefetch_desc(&map_sfq);
        }
    }
    if(warp == 1)
    {
        tmem_alloc(smem_u32(tmem_ptr_smem), static_cast<uint32_t>(prm.tmem_cols));
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    if(threadIdx.x == 0) stamp(1);

    const uint32_t q_box_bytes = static_cast<uint32_t>(bn) * kTileKBytes;
    const uint32_t sfp_bytes   = kScaled ? static_cast<uint32_t>(prm.sf_groups_p) * kSfChunk : 0u;
    const uint32_t sfq_bytes   = kScaled ? static_cast<uint32_t>(prm.sf_groups_q) * kSfChunk : 0u;
    const int nq128            = (bn + 127) / 128;
    const int sfp_cols         = 4 * kAtomsK;
    const int sfq_cols         = 4 * kAtomsK * nq128;

    if(warp == 0)
    {
        // ------------------------------------------------------------------ TMA producer
        if(lane == 0)
        {
            int issued = 0;
            for(int i = 0; i < n_iters; ++i)
            {
                const int s = i % S;
                if(!bounded_wait(empty_bar(s), ((i / S) & 1) ^ 1, abort_f, prm.status, ST_TIMEOUT_PRODUCER, i))
                    break;
                const uint32_t stage = smem_base + s * L.stage_bytes;
                const uint32_t bar   = full_bar(s);
                mbar_arrive_expect_tx(bar, kTileP * kTileKBytes + q_box_bytes + sfp_bytes + sfq_bytes);
                issue_operand_load(prm.p_mode, stage, &map_p, bar, row_p0, it_beg + i);
                issue_operand_load(prm.q_mode, stage + L.q_off, &map_q, bar, row_q0, it_beg + i);
                if(kScaled)
                {
                    tma_load_2d(stage + L.sfp_off, &map_sfp, bar, (it_beg + i) * kSfChunk, row_p0 >> 5);
                    tma_load_2d(stage + L.sfq_off, &map_sfq, bar, (it_beg + i) * kSfChunk, row_q0 >> 5);
                }
                issued = i + 1;
                if(i < 14) stamp(2 + 4 * i);
            }
            if(*abort_f)
            {
                // wait (bounded) for the loads already in flight so that none lands after exit
                for(int i = issued - 1; i >= 0 && i >= issued - S; --i)
                {
                    bool ok = false;
                    const uint64_t t0 = global_timer_ns();
                    while(!ok && global_timer_ns() - t0 < kWaitLimitNs)
                        ok = mbar_try_wait(full_bar(i % S), (i / S) & 1);
                    if(!ok)
                        atomicCAS(prm.status, 0u, ST_TIMEOUT_DRAIN);
                }
            }
        }
    }
    else if(warp == 1)
    {
        // ------------------------------------------------------------------ MMA issuer
        if(lane == 0)
        {
            uint32_t idesc;
            if(KIND == KIND_BF16)
                idesc = idesc_bf16(kTileP, bn);
            else if(KIND == KIND_MXF8)
                idesc = idesc_block_scaled(0, 0, kTileP, bn);
            else
                idesc = idesc_block_scaled(1, 1, kTileP, bn);

            // per-operand descriptor recipe
            const bool p_tiled   = (prm.p_mode == OPM_TILE16);
            const bool q_tiled   = (prm.q_mode == OPM_TILE16);
            const uint32_t p_lbo = p_tiled ? kTileP * 16u : 16u;
            const uint32_t p_sbo = p_tiled ? 128u : 1024u;
            const uint32_t p_lay = p_tiled ? 0u : 2u;
            const uint32_t p_adv = p_tiled ? 2u * kTileP * 16u : 32u; // bytes per 32-byte K step
            const uint32_t q_lbo = q_tiled ? bn * 16u : 16u;
            const uint32_t q_sbo = q_tiled ? 128u : 1024u;
            const uint32_t q_lay = q_tiled ? 0u : 2u;
            const uint32_t q_adv = q_tiled ? 2u * bn * 16u : 32u;

            bool ok = true;
            for(int i = 0; i < n_iters && ok; ++i)
            {
                const int s          = i % S;
                const uint32_t phase = (i / S) & 1;
                ok = bounded_wait(full_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, i);
                if(ok && kScaled)
                    ok = bounded_wait(sf_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_SF, i);
                if(!ok)
                    break;
                tc_fence_after_sync();
                if(i < 14) stamp(5 + 4 * i);
                const uint32_t stage = smem_base + s * L.stage_bytes;
                uint32_t tsfp = 0, tsfq = 0;
                if(kScaled)
                {
                    const uint32_t buf = tmem_base + prm.sf_tmem_base + (i & 1) * (sfp_cols + sfq_cols);
                    tsfp = buf;
                    tsfq = buf + sfp_cols;
                    // scale atoms: P block at sfp_off + a*512 ; Q 128-row block nb at sfq_off + nb*(512*kAtomsK) + a*512
                    for(int a = 0; a < kAtomsK; ++a)
                    {
                        tc_cp_32x128b_warpx4(tsfp + a * 4, make_smem_desc(stage + L.sfp_off + a * 512, 0, 128, 0));
                        for(int nb = 0; nb < nq128; ++nb)
                            tc_cp_32x128b_warpx4(tsfq + (a * nq128 + nb) * 4,
                                                 make_smem_desc(stage + L.sfq_off + nb * (512 * kAtomsK) + a * 512, 0, 128, 0));
                    }
                }
#pragma unroll
                for(int k = 0; k < 4; ++k)
                {
                    const uint64_t pd  = make_smem_desc(stage + k * p_adv, p_lbo, p_sbo, p_lay);
                    const uint64_t qd  = make_smem_desc(stage + L.q_off + k * q_adv, q_lbo, q_sbo, q_lay);
                    const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    if(KIND == KIND_BF16)
                        mma_f16(tmem_base, pd, qd, idesc, acc);
                    else if(KIND == KIND_MXF8)
                        mma_mxf8f6f4(tmem_base, pd, qd, idesc_with_sf(idesc, k, k), acc, tsfp, tsfq);
                    else
                        mma_mxf4(tmem_base, pd, qd, idesc_with_sf(idesc, (k & 1) * 2, (k & 1) * 2), acc,
                                 tsfp + (k >> 1) * 4, tsfq + (k >> 1) * 4 * nq128);
                }
                tc_commit(empty_bar(s));
            }
            stamp(60);
            if(ok)
                tc_commit(accum_bar);
            else
            {
                // abort: let whatever was issued finish before TMEM is released
                tc_commit(drain_bar);
                const uint64_t t0 = global_timer_ns();
                while(!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < kWaitLimitNs) {}
            }
        }
    }
    else if(warp == 2)
    {
        // ------------------------------------------------------------------ scale re-order
        if(kScaled)
        {
            for(int i = 0; i < n_iters; ++i)
            {
                const int s = i % S;
                if(!bounded_wait(full_bar(s), (i / S) & 1, abort_f, prm.status, ST_TIMEOUT_SFWARP, i))
                    break;
                uint8_t* stage = smem_gen + s * L.stage_bytes;
                if(lane == 0 && i < 14) stamp(3 + 4 * i);
                for(int op = 0; op < 2; ++op)
                {
                    uint32_t* region = reinterpret_cast<uint32_t*>(stage + (op == 0 ? L.sfp_off : L.sfq_off));
                    const int groups = (op == 0) ? prm.sf_groups_p : prm.sf_groups_q;
                    const int blocks = (op == 0) ? 1 : nq128;
                    if(SFW == SFW_G1250)
                    {
                        // wire: [group][kq][row 0..31][4 k-blocks]; one atom = 4 groups of one kq
                        // region holds [group][kAtomsK*128 B]
                        for(int nb = 0; nb < blocks; ++nb)
                        {
                            uint32_t w[kAtomsK][4];
#pragma unroll
                            for(int a = 0; a < kAtomsK; ++a)
#pragma unroll
                                for(int g4 = 0; g4 < 4; ++g4)
                                {
                                    const int g = nb * 4 + g4;
                                    w[a][g4]    = (g < groups) ? region[g * (32 * kAtomsK) + a * 32 + lane] : 0x7F7F7F7Fu;
                                }
                            __syncwarp();
#pragma unroll
                            for(int a = 0; a < kAtomsK; ++a)
                                *reinterpret_cast<uint4*>(region + nb * (128 * kAtomsK) + a * 128 + lane * 4) =
                                    make_uint4(w[a][0], w[a][1], w[a][2], w[a][3]);
                            __syncwarp();
                        }
                    }
                    else if(SFW == SFW_E8M0_SHUFFLE)
                    {
                        // wire: per 32-row group and 8 k-blocks a 256-byte chunk with byte offset
                        // (k%4)*64 + (m%16)*4 + ((k%8)/4)*2 + (m%32)/16
                        const int r16 = lane & 15, mh = lane >> 4;
                        for(int nb = 0; nb < blocks; ++nb)
                        {
                            uint32_t w[4][4];
#pragma unroll
                            for(int g4 = 0; g4 < 4; ++g4)
#pragma unroll
                                for(int kk = 0; kk < 4; ++kk)
                                {
                                    const int g = nb * 4 + g4;
                                    w[g4][kk]   = (g < groups) ? region[g * 64 + kk * 16 + r16] : 0x7F7F7F7Fu;
                                }
                            __syncwarp();
#pragma unroll
                            for(int kh = 0; kh < 2; ++kh)
                            {
                                const uint32_t b    = kh * 2 + mh;
                                const uint32_t sel  = b | ((4u + b) << 4);
                                const int first_kb  = (it_beg + i) * 8 + kh * 4;
                                const int valid     = min(max(prm.kblocks - first_kb, 0), 4);
                                const uint32_t mask = valid >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid)) - 1u);
                                uint32_t o[4];
#pragma unroll
                                for(int g4 = 0; g4 < 4; ++g4)
                                {
                                    const uint32_t t01 = __byte_perm(w[g4][0], w[g4][1], sel);
                                    const uint32_t t23 = __byte_perm(w[g4][2], w[g4][3], sel);
                                    const uint32_t v   = __byte_perm(t01, t23, 0x5410);
                                    o[g4]              = (v & mask) | (0x7F7F7F7Fu & ~mask);
                                }
                                *reinterpret_cast<uint4*>(region + nb * 256 + kh * 128 + lane * 4) =
                                    make_uint4(o[0], o[1], o[2], o[3]);
                            }
                            __syncwarp();
                        }
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if(lane == 0)
                {
                    mbar_arrive(sf_bar(s));
                    if(i < 14) stamp(4 + 4 * i);
                }
            }
        }
    }
    else
    {
        // ------------------------------------------------------------------ epilogue (warps 3..6)
        const int quarter = warp & 3; // TMEM lanes 32*quarter .. +31 belong to this warp
        const int p_local = quarter * 32 + lane;
        const int p       = row_p0 + p_local;
        bool ok = bounded_wait(accum_bar, 0, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0);
        ok      = __all_sync(0xffffffffu, ok);
        tc_fence_after_sync();
        if(warp == 3 && lane == 0) stamp(61);
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const int chunk      = bn < 32 ? 16 : 32;
        const int n_chunks   = bn / chunk;
        const bool split     = (splits > 1);
        const int tile_lin   = blockIdx.y * gridDim.x + blockIdx.x;
        bool is_last         = !split;

        if(ok && split)
        {
            float* mine = prm.ws_partial + (static_cast<size_t>(tile_lin) * splits + blockIdx.z) * (static_cast<size_t>(bn) * kTileP);
            for(int c = 0; c < n_chunks; ++c)
            {
                uint32_t r[32];
                if(chunk == 32)
                    tmem_ld_x32(tlane + c * 32, r);
                else
                    tmem_ld_x16(tlane + c * 16, r);
                tmem_ld_wait();
#pragma unroll
                for(int j = 0; j < 32; ++j)
                    if(j < chunk)
                        mine[static_cast<size_t>(c * chunk + j) * kTileP + p_local] = __uint_as_float(r[j]);
            }
            __threadfence();
            // meet the other epilogue warps, take a ticket, meet again (all waits bounded)
            __syncwarp();
            if(lane == 0)
                mbar_arrive(epi_bar);
            ok = bounded_wait(epi_bar, 0, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 1);
            ok = __all_sync(0xffffffffu, ok);
            if(ok)
            {
                if(warp == 3 && lane == 0)
                {
                    *ticket_smem = atomicAdd(prm.ws_counter + tile_lin, 1u);
                    __threadfence_block();
                }
                __syncwarp();
                if(lane == 0)
                    mbar_arrive(epi_bar);
                ok = bounded_wait(epi_bar, 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 2);
                ok = __all_sync(0xffffffffu, ok);
            }
            is_last = ok && (*reinterpret_cast<volatile uint32_t*>(ticket_smem) == static_cast<uint32_t>(splits - 1));
            if(is_last)
                __threadfence();
        }

        if(ok && is_last)
        {
            const float* part = split ? prm.ws_partial + static_cast<size_t>(tile_lin) * splits * (static_cast<size_t>(bn) * kTileP) : nullptr;
            const bool vec_ok = (!prm.transposed_out) && ((prm.ldo & 7) == 0) &&
                                ((reinterpret_cast<uintptr_t>(prm.out) & 15) == 0);
            for(int c = 0; c < n_chunks; ++c)
            {
                float v[32];
                if(!split)
                {
                    uint32_t r[32];
                    if(chunk == 32)
                        tmem_ld_x32(tlane + c * 32, r);
                    else
                        tmem_ld_x16(tlane + c * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                        v[j] = __uint_as_float(r[j]);
                }
                else
                {
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                        v[j] = 0.f;
                    for(int z = 0; z < splits; ++z)
                    {
                        const float* src = part + static_cast<size_t>(z) * (static_cast<size_t>(bn) * kTileP);
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                            if(j < chunk)
                                v[j] += __ldcg(src + static_cast<size_t>(c * chunk + j) * kTileP + p_local);
                    }
                }
                const int q_first = row_q0 + c * chunk;
                // out = alpha * acc + beta * bias
                if(prm.bias != nullptr)
                {
                    const float bp = (!prm.bias_on_q && p < prm.rows_p) ? load_bias(prm.bias, prm.bias_is_bf16, p) : 0.f;
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                    {
                        float b = bp;
                        if(prm.bias_on_q)
                            b = (j < chunk && q_first + j < prm.rows_q) ? load_bias(prm.bias, prm.bias_is_bf16, q_first + j) : 0.f;
                        v[j] = prm.alpha * v[j] + prm.beta * b;
                    }
                }
                else if(prm.alpha != 1.0f)
                {
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                        v[j] *= prm.alpha;
                }

                if(p < prm.rows_p)
                {
                    if(!prm.transposed_out)
                    {
                        __nv_bfloat16* dst = prm.out + static_cast<size_t>(p) * prm.ldo + q_first;
                        if(vec_ok && q_first + chunk <= prm.rows_q)
                        {
#pragma unroll
                            for(int j = 0; j < 32; j += 8)
                                if(j < chunk)
                                {
                                    uint4 o = make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                                                         pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
                                    *reinterpret_cast<uint4*>(dst + j) = o;
                                }
                        }
                        else
                        {
#pragma unroll
                            for(int j = 0; j < 32; ++j)
                                if(j < chunk && q_first + j < prm.rows_q)
                                    dst[j] = __float2bfloat16_rn(v[j]);
                        }
                    }
                    else
                    {
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                        {
                            const int q = q_first + j;
                            if(j < chunk && q < prm.rows_q)
                                prm.out[static_cast<size_t>(q) * prm.ldo + p] = __float2bfloat16_rn(v[j]);
                        }
                    }
                }
            }
            if(split && warp == 3 && lane == 0)
                prm.ws_counter[tile_lin] = 0; // ready for the next launch
        }
        if(warp == 3 && lane == 0) stamp(62);
        tc_fence_before_sync();
    }

    __syncthreads();
    if(threadIdx.x == 0) stamp(63);
    if(warp == 1)
    {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, static_cast<uint32_t>(prm.tmem_cols));
    }
}

} // namespace b200
