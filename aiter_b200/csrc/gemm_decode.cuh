// Decode-shape GEMM (at most 64 activation rows) for sm_100a: a deliberately small kernel.
//
//   D[n][m] = sum_k W[n][k] * X[m][k]      W: 128 weight rows per CTA on the TMEM lanes, X: the M <= 64 activation rows
//                                          on the N side of the MMA (16, 32 or 64 columns); out[m][n] is stored transposed
//
// Why a second kernel beside the persistent one: a decode GEMM moves a few MB and lasts a few microseconds, so what it
// costs is not bytes or flops but the chain of latencies from launch to the last store, paid by single threads.  This
// kernel is built to keep that chain short:
//   * little code: one tile per CTA, one operand arrangement (weights on the 128-row slot), no pairs, no work list, so
//     the lone threads that run each role meet few instruction-cache misses;
//   * 224 threads, <= 146 registers, <= 113 KB of shared memory and <= 256 TMEM columns: two CTAs fit on an SM, so the
//     CTAs of the next launch in the stream (programmatic dependent launch) set up - barriers, TMEM, tensor-map
//     prefetch - while the previous launch still runs, and a grid of up to 296 tiles is one wave;
//   * the four scale warps are also the epilogue warps (same TMEM lane quarters), and one thread issues both operand
//     loads of a K tile;
//   * K split across the CTAs of a cluster (2 or 4) as a reduce-scatter through distributed shared memory, with the
//     cluster barrier split into an early relaxed arrive and a late wait, so nobody idles at a rendezvous.
//
// Warps: 0 operand producer, 1 MMA issuer + TMEM owner, 2..5 scales then epilogue (one per TMEM lane quarter),
//        6 raw-scale producer.  Every barrier wait is bounded (bounded_wait).
#pragma once
#include "gemm_common.cuh"

namespace b200 {

constexpr int kDecodeThreads   = 224;
constexpr int kDecodeMaxStages = 8;

struct DecodeParams
{
    int rows_p, rows_q;      // weight rows (the problem's N), activation rows (the problem's M)
    int num_k_iters;         // ceil(K bytes / 128)
    int kblocks;             // valid 32-element scale blocks along K
    int bn;                  // MMA N: 16, 32, 64 or 128; blockIdx.y counts tiles of bn activation rows (more than one only for bn >= 64)
    int stages;
    int p_mode, q_mode;      // OperandMode of the weights / activations
    int csplit;              // K slices = CTAs per cluster: 1, 2 or 4
    int tma_store;           // the output leaves as per-warp TMA tile stores (map_out is valid)
    int tmem_cols;           // allocation (power of two)
    uint32_t stage_bytes, q_off, sfp_off, sfq_off, cook_off, stg_off, red_off, bar_off;
    int sf_via_cp;           // the scale warps only re-order the scales in shared memory; the MMA thread copies them to TMEM (tcgen05.cp)
    __nv_bfloat16* out;
    long long ldo;
    const void* bias;        // indexed by weight row, or null
    int bias_is_bf16;
    float alpha, beta;
    unsigned int* status;
    unsigned long long* trace; // AITER_B200_TRACING builds only
};

// TMEM columns of one stage's scales: [P atom a: 4 columns][Q atom a: 4 columns], a < atoms per K tile
__host__ __device__ constexpr int decode_sf_cols(int kind)
{
    return kind == KIND_BF16 ? 0 : (kind == KIND_NVF4 ? 32 : (kind == KIND_MXF4 ? 16 : 8));
}
// raw scale bytes per 32-row group per K tile in units of 256 (NVFP4: 512 bytes)
__host__ __device__ constexpr int decode_sf_unit(int kind) { return kind == KIND_BF16 ? 0 : (kind == KIND_NVF4 ? 2 : 1); }
// (the mixed kind, e4m3 activations x packed e2m1 weights, is MXF8 once the scale warps have widened the weight tile to
// e4m3 in shared memory: exact, every e2m1 value is an e4m3 value)

template <int KIND, int SFW>
__global__ void __launch_bounds__(kDecodeThreads, 2)
gemm_decode_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_sfp, const __grid_constant__ CUtensorMap map_sfq,
                   const __grid_constant__ CUtensorMap map_out, const DecodeParams prm)
{
    constexpr bool kScaled = (KIND != KIND_BF16);
    constexpr bool kMixed  = (KIND == KIND_MXF8F4);
    constexpr bool kNvf4   = (KIND == KIND_NVF4);
    constexpr int kAtomsK  = kNvf4 ? 4 : ((KIND == KIND_MXF4) ? 2 : 1); // scale atoms (one 32-bit word per row) per 128-byte K tile
    constexpr uint32_t kNeutralSf = kNvf4 ? 0x38383838u : 0x7F7F7F7Fu; // four scale bytes of 1.0 (e4m3 / e8m0)
    constexpr int kSfCols  = decode_sf_cols(KIND);
    constexpr bool kE8     = (SFW == SFW_E8M0_SHUFFLE);
    constexpr int kSfChunk = kE8 ? 256 : 128 * kAtomsK;   // raw scale bytes per 32-row group per K tile

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const int bn             = prm.bn;
    const int S              = prm.stages;
    const uint32_t bar_base  = smem_base + prm.bar_off;
    auto full_bar            = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar           = [&](int s) { return bar_base + 64u + 8u * s; };
    auto sfraw_bar           = [&](int s) { return bar_base + 128u + 8u * s; };
    const uint32_t acc_bar   = bar_base + 192u;
    const uint32_t red_bar   = bar_base + 200u;
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + prm.bar_off + 208);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + prm.bar_off + 212);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    B200_TRACE(const bool tracing = (prm.trace != nullptr) && blockIdx.x == 0;)
    B200_TRACE(auto stamp = [&](int slot) { if(tracing && slot < 64) prm.trace[slot] = static_cast<unsigned long long>(clock64()); };)
    B200_TRACE(if(threadIdx.x == 0) stamp(0);)
    B200_TRACE(if(prm.trace != nullptr && threadIdx.x == 0 && blockIdx.x < 160) prm.trace[64 + 2 * blockIdx.x] = global_timer_ns();)
    const int csplit     = prm.csplit;
    const uint32_t zrank = csplit > 1 ? cluster_ctarank() : 0u;           // this CTA's K slice
    const int tile       = csplit > 1 ? static_cast<int>(blockIdx.x) / csplit : static_cast<int>(blockIdx.x);
    const int row_p0     = tile * kTileP;
    const int row_q0     = static_cast<int>(blockIdx.y) * bn; // this CTA's activation rows (the same weight tile serves every y)
    const int it_beg     = static_cast<int>(static_cast<uint32_t>(prm.num_k_iters) * zrank / static_cast<uint32_t>(csplit));
    const int n_iters    = static_cast<int>(static_cast<uint32_t>(prm.num_k_iters) * (zrank + 1u) / static_cast<uint32_t>(csplit)) - it_beg;
    const uint32_t per   = static_cast<uint32_t>(kTileP / csplit); // rows of the tile this CTA adds up and stores (whole warps)

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            mbar_init(full_bar(s), kScaled ? 5 : 1); // the operand producer's expect_tx arrival + one arrival per scale warp
            mbar_init(empty_bar(s), 1);
            mbar_init(sfraw_bar(s), kMixed ? 2 : 1); // raw scales (+ the packed e2m1 weight tile of the mixed kind: one wait covers both)
        }
        mbar_init(acc_bar, 1);
        mbar_init(red_bar, 1);
        *abort_f = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
        if(csplit > 1) // the other slices' partial sums of this CTA's rows: posted before anybody can send
            mbar_arrive_expect_tx(red_bar, static_cast<uint32_t>(csplit - 1) * per * static_cast<uint32_t>(bn) * 4u);
    }
    if(warp == 6 && lane == 0)
    {
        tma_prefetch_desc(&map_p);
        tma_prefetch_desc(&map_q);
        if(kScaled)
        {
            tma_prefetch_desc(&map_sfp);
            tma_prefetch_desc(&map_sfq);
        }
        if(prm.tma_store)
            tma_prefetch_desc(&map_out);
    }
    if(warp == 1)
    {
        tmem_alloc(smem_u32(tmem_ptr_smem), static_cast<uint32_t>(prm.tmem_cols));
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    if(csplit > 1)
        cluster_arrive_relaxed(); // "my barriers exist" (made visible by the init fence above); checked before the first remote access
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    B200_TRACE(if(threadIdx.x == 0) stamp(1);)
    // Programmatic dependent launch: everything above may run while the previous kernel of the stream still does;
    // nothing below touches global memory before that kernel has completed.
    grid_dependency_wait();
    grid_launch_dependents();
    B200_TRACE(if(threadIdx.x == 0) stamp(2);)

    if(warp == 0)
    {
        // ------------------------------------------------------------------ operand producer
        if(lane == 0)
        {
            const uint32_t q_bytes = static_cast<uint32_t>(bn) * kTileKBytes;
            int s = 0;
            uint32_t phase = 0;
            int kt = it_beg;
            for(int i = 0; i < n_iters; ++i, ++kt)
            {
                if(!bounded_wait(empty_bar(s), phase ^ 1u, abort_f, prm.status, ST_TIMEOUT_PRODUCER, i))
                    break;
                const uint32_t stage = smem_base + s * prm.stage_bytes;
                const uint32_t bar   = full_bar(s);
                if(kMixed)
                {
                    // the packed e2m1 weight tile (16x16-byte tiled: 4 chunks of 16 bytes = 32 codes per row) lands in the
                    // staging area and is counted on the raw-scale barrier, which the widening warps wait on
                    mbar_arrive_expect_tx(sfraw_bar(s), kTileP * 64u);
                    tma_load_3d(stage + prm.stg_off, &map_p, sfraw_bar(s), 0, row_p0 >> 4, kt * 4);
                    mbar_arrive_expect_tx(bar, q_bytes);
                }
                else
                {
                    mbar_arrive_expect_tx(bar, kTileP * kTileKBytes + q_bytes);
                    issue_operand_load(prm.p_mode, stage, &map_p, bar, row_p0, kt);
                }
                issue_operand_load(prm.q_mode, stage + prm.q_off, &map_q, bar, row_q0, kt);
                B200_TRACE(if(i == 0) stamp(3);)
                if(++s == S)
                {
                    s = 0;
                    phase ^= 1u;
                }
            }
            if(*abort_f)
            {
                // give loads still in flight time to land before this CTA's shared memory is released (bounded)
                const uint64_t t0 = global_timer_ns();
                while(global_timer_ns() - t0 < 200000ull) {}
            }
        }
    }
    else if(warp == 6)
    {
        // ------------------------------------------------------------------ raw scale producer
        // (test hook: with c_wait_ctl.withhold_scales set this role issues nothing, so the waits behind it run out)
        if(kScaled && lane == 0 && c_wait_ctl.withhold_scales == 0u)
        {
            const uint32_t sfp_bytes = 4u * kSfChunk;
            const uint32_t sfq_bytes = static_cast<uint32_t>((bn + 31) / 32) * kSfChunk;
            int s = 0;
            uint32_t phase = 0;
            int kc = it_beg * kSfChunk;
            for(int i = 0; i < n_iters; ++i, kc += kSfChunk)
            {
                if(!bounded_wait(empty_bar(s), phase ^ 1u, abort_f, prm.status, ST_TIMEOUT_PRODUCER, 0x20000 + i))
                    break;
                const uint32_t stage = smem_base + s * prm.stage_bytes;
                const uint32_t bar   = sfraw_bar(s);
                mbar_arrive_expect_tx(bar, sfp_bytes + sfq_bytes);
                if(kNvf4) // 512-byte chunks are two 256-byte pieces of a 3-D view (a box dimension holds 256 elements)
                {
                    tma_load_3d(stage + prm.sfp_off, &map_sfp, bar, 0, kc >> 8, row_p0 >> 5);
                    tma_load_3d(stage + prm.sfq_off, &map_sfq, bar, 0, kc >> 8, row_q0 >> 5);
                }
                else
                {
                    tma_load_2d(stage + prm.sfp_off, &map_sfp, bar, kc, row_p0 >> 5);
                    tma_load_2d(stage + prm.sfq_off, &map_sfq, bar, kc, row_q0 >> 5);
                }
                if(++s == S)
                {
                    s = 0;
                    phase ^= 1u;
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
            else if(KIND == KIND_MXF8 || KIND == KIND_MXF8F4)
                idesc = idesc_block_scaled(0, 0, kTileP, bn);
            else
                idesc = idesc_block_scaled(1, 1, kTileP, bn, !kNvf4);
            const bool p_tiled   = (prm.p_mode == OPM_TILE16);
            const bool q_tiled   = (prm.q_mode == OPM_TILE16);
            const uint32_t p_lbo = p_tiled ? kTileP * 16u : 16u, p_sbo = p_tiled ? 128u : 1024u, p_lay = p_tiled ? 0u : 2u;
            const uint32_t q_lbo = q_tiled ? bn * 16u : 16u, q_sbo = q_tiled ? 128u : 1024u, q_lay = q_tiled ? 0u : 2u;
            const uint32_t p_step = (p_tiled ? 2u * kTileP * 16u : 32u) >> 4;
            const uint32_t q_step = (q_tiled ? 2u * bn * 16u : 32u) >> 4;
            // descriptor words once; per MMA only an add on the address field (this thread pays every instruction's latency)
            const uint32_t p_hi  = static_cast<uint32_t>(make_smem_desc(0, p_lbo, p_sbo, p_lay) >> 32);
            const uint32_t q_hi  = static_cast<uint32_t>(make_smem_desc(0, q_lbo, q_sbo, q_lay) >> 32);
            const uint32_t p_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base, p_lbo, p_sbo, p_lay));
            const uint32_t q_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base + prm.q_off, q_lbo, q_sbo, q_lay));
            const uint32_t stage_step = prm.stage_bytes >> 4;
            // re-ordered scales: 32 rows of 16 bytes, 8-row groups 128 bytes apart, no swizzle
            const uint32_t cook_hi  = static_cast<uint32_t>(make_smem_desc(0, 16u, 128u, 0u) >> 32);
            const uint32_t cook_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base + prm.cook_off, 16u, 128u, 0u));
            uint32_t idk[4];
#pragma unroll
            for(int k = 0; k < 4; ++k)
                idk[k] = (KIND == KIND_BF16 || kNvf4) ? idesc
                         : (KIND == KIND_MXF4)        ? idesc_with_sf(idesc, (k & 1) * 2, (k & 1) * 2)
                                                      : idesc_with_sf(idesc, k, k);
            const uint32_t sf0 = tmem_base + bn; // the scale buffers follow the accumulator (bn columns)
            bool ok = true;
            int s = 0;
            uint32_t phase = 0;
            for(int i = 0; i < n_iters; ++i)
            {
                ok = bounded_wait(full_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, i);
                if(!ok)
                    break;
                tc_fence_after_sync();
                B200_TRACE(if(i < 8) stamp(4 + i);)
                const uint32_t p_lo = p_lo0 + s * stage_step;
                const uint32_t q_lo = q_lo0 + s * stage_step;
                const uint32_t tsfp = sf0 + s * kSfCols;
                const uint32_t tsfq = tsfp + 4 * kAtomsK;
                if(kScaled && prm.sf_via_cp)
                {
                    // the stage's re-ordered scales: per K atom 32 rows x 16 bytes for the weights and as much for the
                    // activations, copied to TMEM and replicated over the four lane quarters by the tensor core's own copy
                    // unit; issued by this thread right before the MMAs that read them, which the pipe keeps in order
                    const uint32_t c_lo = cook_lo0 + s * stage_step;
#pragma unroll
                    for(int a = 0; a < kAtomsK; ++a)
                    {
                        tc_cp_32x128b_warpx4(tsfp + a * 4, pack_u64(c_lo + a * 32u, cook_hi));
                        tc_cp_32x128b_warpx4(tsfq + a * 4, pack_u64(c_lo + (kAtomsK + a) * 32u, cook_hi));
                    }
                }
#pragma unroll
                for(int k = 0; k < 4; ++k)
                {
                    const uint64_t pd  = pack_u64(p_lo + k * p_step, p_hi);
                    const uint64_t qd  = pack_u64(q_lo + k * q_step, q_hi);
                    const uint32_t acc = (k > 0) ? 1u : static_cast<uint32_t>(i > 0);
                    if(KIND == KIND_BF16)
                        mma_f16(tmem_base, pd, qd, idk[k], acc);
                    else if(KIND == KIND_MXF8 || KIND == KIND_MXF8F4)
                        mma_mxf8f6f4(tmem_base, pd, qd, idk[k], acc, tsfp, tsfq);
                    else if(kNvf4)
                        mma_nvf4(tmem_base, pd, qd, idk[k], acc, tsfp + k * 4, tsfq + k * 4);
                    else
                        mma_mxf4(tmem_base, pd, qd, idk[k], acc, tsfp + (k >> 1) * 4, tsfq + (k >> 1) * 4);
                }
                tc_commit(empty_bar(s));
                if(++s == S)
                {
                    s = 0;
                    phase ^= 1u;
                }
            }
            if(ok)
                tc_commit(acc_bar);
            B200_TRACE(stamp(30);)
        }
    }
    else
    {
        // ------------------------------------------------------------------ warps 2..5: scales, then the epilogue
        const int quarter    = warp & 3;
        const int p_local    = quarter * 32 + lane;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        bool ok = true;
        if(kScaled)
        {
            const int q_groups = (bn + 31) / 32; // 1 to 4 groups of 32 activation rows (the weights always stage 4)
            const int r16 = lane & 15, hi = lane >> 4;
            int s = 0;
            uint32_t phase = 0;
            int kt = it_beg;
            for(int i = 0; i < n_iters && ok; ++i, ++kt)
            {
                ok = bounded_wait(sfraw_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_SFWARP, i);
                ok = __all_sync(0xffffffffu, ok);
                if(!ok)
                    break;
                B200_TRACE(if(warp == 2 && lane == 0 && i < 8) stamp(12 + i);)
                const uint8_t* stage = smem_gen + s * prm.stage_bytes;
                if(kMixed)
                {
                    // widen this thread's weight row: 4 chunks of 32 packed codes -> 8 chunks of 16 e4m3 bytes, in the
                    // un-swizzled K-major layout the MMA reads ([chunk][row][16 B]); all loads first so their latencies overlap
                    const int t_row  = (warp - 2) * 32 + lane;
                    const uint4* src = reinterpret_cast<const uint4*>(stage + prm.stg_off);
                    uint4* dst       = reinterpret_cast<uint4*>(smem_gen + s * prm.stage_bytes);
                    uint4 v[4];
#pragma unroll
                    for(int c = 0; c < 4; ++c)
                        v[c] = src[c * kTileP + t_row];
#pragma unroll
                    for(int c = 0; c < 4; ++c)
                    {
                        uint4 o0, o1;
                        e2m1x8_to_e4m3x8(v[c].x, o0.x, o0.y);
                        e2m1x8_to_e4m3x8(v[c].y, o0.z, o0.w);
                        e2m1x8_to_e4m3x8(v[c].z, o1.x, o1.y);
                        e2m1x8_to_e4m3x8(v[c].w, o1.z, o1.w);
                        dst[(2 * c) * kTileP + t_row]     = o0;
                        dst[(2 * c + 1) * kTileP + t_row] = o1;
                    }
                    fence_proxy_async_smem(); // read by the tensor core
                }
                if(prm.sf_via_cp)
                {
                    // This warp re-orders only its share of the groups (warp w: group w of the weights and, if there is
                    // one, group w of the activations) and leaves the result where the MMA thread's tcgen05.cp finds it:
                    // cooked[K atom a][row 0..31][group g] words for the weights, then the same for the activations.
                    uint32_t* cooked = reinterpret_cast<uint32_t*>(smem_gen + s * prm.stage_bytes + prm.cook_off);
                    const int wq     = warp - 2;
#pragma unroll
                    for(int side = 0; side < 2; ++side)
                    {
                        if(side == 1 && wq >= q_groups)
                            break;
                        uint32_t* dst = cooked + (side ? kAtomsK * 128 : 0) + lane * 4 + wq;
                        if(kE8)
                        {
                            const uint32_t* grp = reinterpret_cast<const uint32_t*>(stage + (side ? prm.sfq_off : prm.sfp_off) + wq * 256);
                            const uint32_t w0 = grp[r16], w1 = grp[16 + r16], w2 = grp[32 + r16], w3 = grp[48 + r16];
                            const uint32_t sel     = hi ? 0x7351u : 0x6240u;
                            const uint32_t lo_part = __byte_perm(w0, w1, sel);
                            const uint32_t hi_part = __byte_perm(w2, w3, sel);
                            uint32_t v0 = __byte_perm(lo_part, hi_part, 0x5410);
                            uint32_t v1 = __byte_perm(lo_part, hi_part, 0x7632);
                            if(kt * 8 + 8 > prm.kblocks)
                            {
                                const int valid0  = min(max(prm.kblocks - kt * 8, 0), 4);
                                const int valid1  = min(max(prm.kblocks - kt * 8 - 4, 0), 4);
                                const uint32_t m0 = valid0 >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid0)) - 1u);
                                const uint32_t m1 = valid1 >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid1)) - 1u);
                                v0 = (v0 & m0) | (0x7F7F7F7Fu & ~m0);
                                v1 = (v1 & m1) | (0x7F7F7F7Fu & ~m1);
                            }
                            dst[0] = v0;
                            if(kAtomsK == 2)
                                dst[128] = v1;
                        }
                        else
                        {
                            const uint32_t* grp = reinterpret_cast<const uint32_t*>(stage + (side ? prm.sfq_off : prm.sfp_off) + wq * kSfChunk);
#pragma unroll
                            for(int a = 0; a < kAtomsK; ++a)
                                dst[a * 128] = grp[a * 32 + lane];
                        }
                    }
                    fence_proxy_async_smem(); // read by the tensor core's copy unit
                    __syncwarp();
                    if(lane == 0)
                        mbar_arrive(full_bar(s));
                    B200_TRACE(if(warp == 2 && lane == 0 && i < 8) stamp(20 + i);)
                    if(++s == S)
                    {
                        s = 0;
                        phase ^= 1u;
                    }
                    continue;
                }
                uint32_t t[kSfCols > 0 ? kSfCols : 1];
#pragma unroll
                for(int c = 0; c < kSfCols; ++c)
                    t[c] = kNeutralSf;
                if(kE8)
                {
                    // raw: per 32-row group j a 256-byte chunk, byte (k%4)*64 + (m%16)*4 + ((k%8)/4)*2 + (m%32)/16: this lane's
                    // row has its eight scale bytes in four words (one per k%4), at byte kh*2 + (row half)
                    const bool tail    = (kt * 8 + 8 > prm.kblocks);
                    const uint32_t sel = hi ? 0x7351u : 0x6240u;
                    uint32_t raw[8][4];
#pragma unroll
                    for(int j = 0; j < 8; ++j)
                    {
                        const uint32_t* grp = reinterpret_cast<const uint32_t*>(stage + (j < 4 ? prm.sfp_off + j * 256 : prm.sfq_off + (j - 4) * 256));
#pragma unroll
                        for(int c = 0; c < 4; ++c)
                            raw[j][c] = (j < 4 + q_groups) ? grp[c * 16 + r16] : 0u;
                    }
#pragma unroll
                    for(int j = 0; j < 8; ++j)
                    {
                        const uint32_t lo_part = __byte_perm(raw[j][0], raw[j][1], sel); // k%4 = 0,1 for both k halves
                        const uint32_t hi_part = __byte_perm(raw[j][2], raw[j][3], sel); // k%4 = 2,3
                        uint32_t v0 = __byte_perm(lo_part, hi_part, 0x5410);             // k-blocks 0..3 of this row
                        uint32_t v1 = __byte_perm(lo_part, hi_part, 0x7632);             // k-blocks 4..7
                        if(tail)
                        {
                            // scale bytes beyond K read as 2^0 (their data bytes are zero-filled by the tile loads)
                            const int valid0  = min(max(prm.kblocks - kt * 8, 0), 4);
                            const int valid1  = min(max(prm.kblocks - kt * 8 - 4, 0), 4);
                            const uint32_t m0 = valid0 >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid0)) - 1u);
                            const uint32_t m1 = valid1 >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid1)) - 1u);
                            v0 = (v0 & m0) | (0x7F7F7F7Fu & ~m0);
                            v1 = (v1 & m1) | (0x7F7F7F7Fu & ~m1);
                        }
                        if(j < 4 + q_groups && kAtomsK == 2)
                        {
                            t[(j < 4) ? j : 8 + (j - 4)]      = v0; // K atom 0: P columns 0..3, Q columns 8..11
                            t[(j < 4) ? 4 + j : 12 + (j - 4)] = v1; // K atom 1: P columns 4..7, Q columns 12..15
                        }
                    }
                }
                else if(kNvf4)
                {
                    // raw: [group][wire tile h = 0, 1][row 0..31][8 scales]: two words per row per wire tile, K atoms 2h and 2h + 1
#pragma unroll
                    for(int j = 0; j < 8; ++j)
#pragma unroll
                        for(int h = 0; h < 2; ++h)
                        {
                            const uint2* grp = reinterpret_cast<const uint2*>(stage + (j < 4 ? prm.sfp_off + j * 512 : prm.sfq_off + (j - 4) * 512));
                            if(j < 4 + q_groups)
                            {
                                const uint2 v = grp[h * 32 + lane];
                                t[(j < 4) ? (2 * h) * 4 + j : 16 + (2 * h) * 4 + (j - 4)]         = v.x;
                                t[(j < 4) ? (2 * h + 1) * 4 + j : 16 + (2 * h + 1) * 4 + (j - 4)] = v.y;
                            }
                        }
                }
                else
                {
                    // raw: [group][K atom a][row 0..31][4 k-blocks]: one word per row per K atom
#pragma unroll
                    for(int j = 0; j < 8; ++j)
#pragma unroll
                        for(int a = 0; a < kAtomsK; ++a)
                        {
                            const uint32_t* grp = reinterpret_cast<const uint32_t*>(stage + (j < 4 ? prm.sfp_off + j * kSfChunk : prm.sfq_off + (j - 4) * kSfChunk));
                            const int col       = (j < 4) ? a * 4 + j : 4 * kAtomsK + a * 4 + (j - 4);
                            if(j < 4 + q_groups)
                                t[col] = grp[a * 32 + lane];
                        }
                }
                const uint32_t tsf = tlane + bn + s * kSfCols;
                if(kSfCols == 32)
                {
                    tmem_st_x16(tsf, t);
                    tmem_st_x16(tsf + 16, t + 16);
                }
                else if(kSfCols == 16)
                    tmem_st_x16(tsf, t);
                else
                    tmem_st_x8(tsf, t);
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if(lane == 0)
                    mbar_arrive(full_bar(s));
                B200_TRACE(if(warp == 2 && lane == 0 && i < 8) stamp(20 + i);)
                if(++s == S)
                {
                    s = 0;
                    phase ^= 1u;
                }
            }
        }

        // ---- epilogue: this thread holds row p_local of the tile (one weight row = one output column), bn values
        // (the cluster check sits here, in the slack while the last K tile's MMAs run: every CTA of the cluster has
        // initialised its barriers - they all ran a K loop since - before this CTA touches their shared memory)
        if(csplit > 1)
            cluster_wait_acquire();
        if(ok)
        {
            ok = bounded_wait(acc_bar, 0, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0);
            ok = __all_sync(0xffffffffu, ok);
        }
        B200_TRACE(if(lane == 0) stamp(38 + (warp - 2));)
        if(ok)
        {
            tc_fence_after_sync();
            // the thread's row goes out in chunks of at most 64 columns (one chunk unless bn = 128)
            const int n_chunks = (bn + 63) >> 6;
            for(int h = 0; h < n_chunks && ok; ++h)
            {
            const int c0 = h * 64;                  // first column (activation row of the tile) of this chunk
            const int bw = min(bn - c0, 64);        // its width: 16, 32 or 64
            float v[64];
            {
                uint32_t r[32] = {};
                if(bw == 16)
                    tmem_ld_x16(tlane + c0, r);
                else
                    tmem_ld_x32(tlane + c0, r);
                tmem_ld_wait();
#pragma unroll
                for(int j = 0; j < 32; ++j)
                    v[j] = __uint_as_float(r[j]);
                if(bw == 64)
                {
                    tmem_ld_x32(tlane + c0 + 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                        v[32 + j] = __uint_as_float(r[j]);
                }
            }
            bool mine = true; // this warp adds up and stores its rows
            if(csplit > 1)
            {
                // Reduce-scatter over the cluster: CTA z owns rows [z * per, (z + 1) * per) of the tile (whole warps).  A warp
                // whose rows belong to another CTA sends its partial sums to that CTA's shared memory ([source slice][row][bn
                // floats], bytes counted on that CTA's red barrier) and is done; an owning warp waits for the other slices
                // (once: the barrier counts the bytes of every chunk).
                const uint32_t owner = static_cast<uint32_t>(p_local) / per;
                const uint32_t prow  = static_cast<uint32_t>(p_local) - owner * per;
                mine                 = (owner == zrank);
                if(!mine)
                {
                    const uint32_t src     = zrank < owner ? zrank : zrank - 1u; // this slice's place among the owner's sources
                    const uint32_t dst_row = map_to_cta(smem_base + prm.red_off, owner) +
                                             ((src * per + prow) * static_cast<uint32_t>(bn) + static_cast<uint32_t>(c0)) * 4u;
                    const uint32_t dst_bar = map_to_cta(red_bar, owner);
#pragma unroll
                    for(int j = 0; j < 64; j += 4)
                        if(j < bw)
                            st_async_v4(dst_row + static_cast<uint32_t>(j) * 4u, __float_as_uint(v[j]), __float_as_uint(v[j + 1]),
                                        __float_as_uint(v[j + 2]), __float_as_uint(v[j + 3]), dst_bar);
                }
                else
                {
                    if(h == 0)
                    {
                        ok = bounded_wait(red_bar, 0, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x3000);
                        ok = __all_sync(0xffffffffu, ok);
                    }
                    if(ok)
                    {
                        const float4* red = reinterpret_cast<const float4*>(smem_gen + prm.red_off);
                        for(int z = 0; z < csplit - 1; ++z)
                        {
                            const float4* row = red + (static_cast<size_t>(z * per + prow) * bn + c0) / 4;
#pragma unroll
                            for(int j = 0; j < 64; j += 4)
                                if(j < bw)
                                {
                                    const float4 t = row[j / 4];
                                    v[j] += t.x;
                                    v[j + 1] += t.y;
                                    v[j + 2] += t.z;
                                    v[j + 3] += t.w;
                                }
                        }
                    }
                }
            }
            B200_TRACE(if(lane == 0 && h == 0) stamp(42 + (warp - 2));)
            if(ok && mine)
            {
                const int p = row_p0 + p_local;
                if(prm.bias != nullptr)
                {
                    const float b = (p < prm.rows_p) ? prm.beta * load_bias(prm.bias, prm.bias_is_bf16, p) : 0.f;
#pragma unroll
                    for(int j = 0; j < 64; ++j)
                        if(j < bw)
                            v[j] = prm.alpha * v[j] + b;
                }
                else if(prm.alpha != 1.0f)
                {
#pragma unroll
                    for(int j = 0; j < 64; ++j)
                        if(j < bw)
                            v[j] *= prm.alpha;
                }
                if(prm.tma_store)
                {
                    // this warp's 32 output columns x bw rows, staged as [row m][32 x bf16] in a retired operand stage (every
                    // tile load has landed and been consumed once the accumulator is complete; a buffer per warp and chunk)
                    // and stored as one TMA tile, which clips rows >= M and columns >= N
                    const uint32_t buf_off = static_cast<uint32_t>((warp - 2) * 2 + h) * 4096u;
                    uint8_t* buf           = smem_gen + buf_off;
#pragma unroll
                    for(int j = 0; j < 64; ++j)
                        if(j < bw)
                            reinterpret_cast<__nv_bfloat16*>(buf)[j * 32 + lane] = __float2bfloat16_rn(v[j]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    const int p_warp0 = row_p0 + quarter * 32;
                    if(lane == 0 && p_warp0 < prm.rows_p)
                    {
                        tma_store_2d(&map_out, smem_base + buf_off, p_warp0 * 2, row_q0 + c0);
                        bulk_commit_group();
                        bulk_wait_group_read<0>(); // the store has read its source before the CTA retires
                    }
                }
                else if(p < prm.rows_p)
                {
                    // (output whose pitch or base rules out a tensor map; measured 1 to 1.5 us slower per call than the
                    // tile store even for one activation row: plain stores take longer to drain at the grid's end, and the
                    // dependent launch waits for that)
#pragma unroll
                    for(int j = 0; j < 64; ++j)
                        if(j < bw && row_q0 + c0 + j < prm.rows_q)
                            prm.out[static_cast<size_t>(row_q0 + c0 + j) * prm.ldo + p] = __float2bfloat16_rn(v[j]);
                }
            }
            } // chunks of 64 columns
        }
        B200_TRACE(if(lane == 0) stamp(46 + (warp - 2));)
        tc_fence_before_sync();
    }

    __syncthreads();
    B200_TRACE(if(threadIdx.x == 0) stamp(63);)
    B200_TRACE(if(prm.trace != nullptr && threadIdx.x == 0 && blockIdx.x < 160) prm.trace[65 + 2 * blockIdx.x] = global_timer_ns();)
    // no cluster rendezvous at the end: the only remote traffic into a CTA are the partial sums of the rows it owns, and
    // the warps that own them have waited for every byte (red barrier) before the CTA gets here
    if(warp == 1)
    {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, static_cast<uint32_t>(prm.tmem_cols));
    }
}

} // namespace b200
