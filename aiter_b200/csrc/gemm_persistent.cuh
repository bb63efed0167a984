// Persistent warp-specialised tcgen05 GEMM for sm_100a, optionally on CTA pairs (cta_group::2).
//
//   D[p][q] = sum_k P[p][k] * Q[q][k]      P: 128 rows per CTA on the TMEM lanes, Q: BN columns
//
// One CTA (CG = 1) or one pair of CTAs on neighbouring SMs (CG = 2) walks a static list of work units
// (output tile x K split).  In a pair every CTA stages its own 128 rows of P and its own half of the BN
// rows of Q; the leader's MMA thread issues 256 x BN instructions that read both CTAs' shared memory, so
// each SM moves 2/3 of the bytes per flop of the single-CTA tile.  No TMA multicast is used anywhere:
// every CTA fetches exactly the bytes it stages.
//
// Warps (320 threads per CTA):
//   0      TMA producer: operand tiles + raw scale bytes into a ring of shared-memory stages
//   1      MMA issuer (leader CTA) and TMEM owner; in a pair's second CTA it forwards "stage landed"
//   2..5   scale warps: read the raw scale bytes of a stage (any wire layout), re-order them in registers
//          and write them to TMEM with tcgen05.st, one warp per TMEM lane quarter
//   6..9   epilogue: TMEM -> registers -> alpha/bias -> bf16 -> global (or split-K partials + last-arriver
//          reduction), overlapped with the next unit's main loop when two accumulators fit in TMEM
//
// Barriers (all waits bounded by wall time):
//   full[s]       stage s of THIS CTA has landed (TMA transaction bytes)
//   ready[s]      leader only: scale warps of all CTAs have written stage s's scales to TMEM (scaled kinds),
//                 or the second CTA's stage s has landed (bf16 pair)
//   empty[s]      the MMAs reading stage s (and its TMEM scales) are done (tcgen05.commit, both CTAs)
//   acc_full[a]   accumulator a is complete (tcgen05.commit, both CTAs)
//   acc_empty[a]  leader only: all epilogue warps of all CTAs have drained accumulator a
#pragma once
#include "gemm_common.cuh"

namespace b200 {

constexpr int kPersistentThreads = 320;
constexpr int kMaxAcc            = 2;

struct PersistentParams
{
    int rows_p, rows_q;
    int num_k_iters;  // ceil(K bytes / 128)
    int kblocks;      // valid 32-element scale blocks along K
    int bn;           // UMMA N (multiple of 16, <= 256; multiple of 32 unless there is a single Q tile)
    int stages;
    int p_mode, q_mode;
    int sf_groups_p, sf_groups_q; // 32-row scale groups staged per CTA per stage
    int f4_operand;               // mixed kind only: which operand arrives as packed e2m1 (1 = P, 2 = Q)
    int transposed_out;
    int tiles_p, tiles_q, splits; // tiles_p counts 128*CG-row tiles
    int n_acc;                    // accumulators in TMEM (1 or 2)
    int acc_stride;               // TMEM columns between accumulators
    int sf_tmem_base;             // first TMEM column of the per-stage scale buffers
    int sf_cols;                  // TMEM columns per stage for scales
    int tmem_cols;                // allocation (power of two)
    __nv_bfloat16* out;
    long long ldo;
    const void* bias;
    int bias_is_bf16;
    int bias_on_q;
    float alpha, beta;
    float* ws_partial;
    unsigned int* ws_counter;
    unsigned int* status;
    unsigned long long* trace;
};

struct PersistentSmem
{
    uint32_t stage_bytes, q_off, sfp_off, sfq_off, stg_off, bar_off, total;
};

// f4_operand: 0 none, 1 = P, 2 = Q arrives as packed e2m1 and needs a staging area of rows x 64 bytes
__host__ __device__ inline PersistentSmem make_persistent_smem(int kind, int bn, int cg, int stages, int f4_operand = 0)
{
    PersistentSmem L;
    uint32_t q_bytes = static_cast<uint32_t>(bn / cg) * kTileKBytes;
    q_bytes          = (q_bytes + 1023u) & ~1023u;
    L.q_off          = kTileP * kTileKBytes;
    L.sfp_off        = L.q_off + q_bytes;
    L.sfq_off        = L.sfp_off + (kind == KIND_BF16 ? 0u : 1024u);
    L.stg_off        = L.sfq_off + (kind == KIND_BF16 ? 0u : 2048u);
    uint32_t stg     = f4_operand == 1 ? kTileP * 64u : (f4_operand == 2 ? static_cast<uint32_t>(bn / cg) * 64u : 0u);
    stg              = (stg + 1023u) & ~1023u;
    L.stage_bytes    = L.stg_off + stg;
    L.bar_off        = L.stage_bytes * static_cast<uint32_t>(stages);
    L.total          = L.bar_off + 512u;
    return L;
}

// 8 packed e2m1 codes (one 32-bit word, element n in nibble n) -> 8 e4m3 bytes (exact: every e2m1 value
// is an e4m3 value).  Magnitude by table look-up (prmt), sign moved to bit 7 of each byte.
__device__ __forceinline__ void e2m1x8_to_e4m3x8(uint32_t w, uint32_t& lo, uint32_t& hi)
{
    constexpr uint32_t kLutLo = 0x3C383000u; // 0, 0.5, 1, 1.5
    constexpr uint32_t kLutHi = 0x4C484440u; // 2, 3, 4, 6
    constexpr uint32_t kSign  = 0x00008000u; // byte 0 = 0x00, byte 1 = 0x80
    lo = __byte_perm(kLutLo, kLutHi, w & 0x7777u) | __byte_perm(kSign, 0u, (w >> 3) & 0x1111u);
    const uint32_t h = w >> 16;
    hi = __byte_perm(kLutLo, kLutHi, h & 0x7777u) | __byte_perm(kSign, 0u, (h >> 3) & 0x1111u);
}

template <int KIND, int SFW, int CG>
__global__ void __launch_bounds__(kPersistentThreads, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_sfp, const __grid_constant__ CUtensorMap map_sfq,
                       const PersistentParams prm)
{
    constexpr bool kScaled = (KIND != KIND_BF16);
    constexpr bool kMixed  = (KIND == KIND_MXF8F4);
    constexpr int kAtomsK  = (KIND == KIND_MXF4) ? 2 : 1;
    constexpr int kSfChunk = (SFW == SFW_E8M0_SHUFFLE) ? 256 : 128 * kAtomsK;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const int bn             = prm.bn;
    const int S              = prm.stages;
    const PersistentSmem L   = make_persistent_smem(KIND, bn, CG, S, kMixed ? prm.f4_operand : 0);

    const uint32_t bar_base  = smem_base + L.bar_off;
    auto full_bar            = [&](int s) { return bar_base + 8u * s; };
    auto ready_bar           = [&](int s) { return bar_base + 64u + 8u * s; };
    auto empty_bar           = [&](int s) { return bar_base + 128u + 8u * s; };
    auto acc_full_bar        = [&](int a) { return bar_base + 192u + 8u * a; };
    auto acc_empty_bar       = [&](int a) { return bar_base + 208u + 8u * a; };
    const uint32_t epi_bar   = bar_base + 224u;
    const uint32_t drain_bar = bar_base + 232u;
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + L.bar_off + 240);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + L.bar_off + 244);
    uint32_t* ticket_smem      = reinterpret_cast<uint32_t*>(smem_gen + L.bar_off + 248);

    const int warp       = threadIdx.x >> 5;
    const int lane       = threadIdx.x & 31;
    const uint32_t crank = (CG == 2) ? cluster_ctarank() : 0u; // 0 = leader
    const bool leader    = (crank == 0);
    const int cluster_id = blockIdx.x / CG;
    const int n_clusters = gridDim.x / CG;

    const bool tracing = (prm.trace != nullptr) && blockIdx.x == 0;
    auto stamp = [&](int slot) { if(tracing && slot < 64) prm.trace[slot] = static_cast<unsigned long long>(clock64()); };
    if(threadIdx.x == 0) stamp(0);

    const int splits      = prm.splits;
    const int total_units = prm.tiles_p * prm.tiles_q * splits;
    // ready[s] arrivals per phase: scaled kinds - one per scale warp of every CTA; bf16 pair - the second CTA
    const int ready_count = kScaled ? 4 * CG : (CG - 1);

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            mbar_init(full_bar(s), 1);
            mbar_init(ready_bar(s), ready_count > 0 ? ready_count : 1);
            mbar_init(empty_bar(s), 1);
        }
        for(int a = 0; a < kMaxAcc; ++a)
        {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 4 * CG);
        }
        mbar_init(epi_bar, 4);
        mbar_init(drain_bar, 1);
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
        if(CG == 2)
        {
            tmem_alloc_2cta(smem_u32(tmem_ptr_smem), static_cast<uint32_t>(prm.tmem_cols));
            tmem_relinquish_2cta();
        }
        else
        {
            tmem_alloc(smem_u32(tmem_ptr_smem), static_cast<uint32_t>(prm.tmem_cols));
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if(CG == 2)
        cluster_sync_all(); // the partner's barriers exist before anything arrives on them remotely
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    if(threadIdx.x == 0) stamp(1);

    const int q_rows_cta       = bn / CG;
    const uint32_t q_box_bytes = static_cast<uint32_t>(q_rows_cta) * kTileKBytes;
    const uint32_t sfp_bytes   = kScaled ? static_cast<uint32_t>(prm.sf_groups_p) * kSfChunk : 0u;
    const uint32_t sfq_bytes   = kScaled ? static_cast<uint32_t>(prm.sf_groups_q) * kSfChunk : 0u;
    const int nq128            = (bn + 127) / 128;
    const int sfp_cols         = 4 * kAtomsK;

    // unit -> (tile_p, tile_q, k range); q runs fastest so that concurrently running CTAs share P tiles
    auto decode = [&](int u, int& tp, int& tq, int& it_beg, int& n_iters, int& z) {
        z              = u % splits;
        const int tile = u / splits;
        tq             = tile % prm.tiles_q;
        tp             = tile / prm.tiles_q;
        it_beg         = static_cast<int>((static_cast<long long>(prm.num_k_iters) * z) / splits);
        n_iters        = static_cast<int>((static_cast<long long>(prm.num_k_iters) * (z + 1)) / splits) - it_beg;
    };

    if(warp == 0)
    {
        // ------------------------------------------------------------------ TMA producer (every CTA)
        if(lane == 0)
        {
            int g = 0; // running stage counter
            bool ok = true;
            for(int u = cluster_id; u < total_units && ok; u += n_clusters)
            {
                int tp, tq, it_beg, n_iters, z;
                decode(u, tp, tq, it_beg, n_iters, z);
                const int row_p0 = (tp * CG + static_cast<int>(crank)) * kTileP;
                const int row_q0 = tq * bn + static_cast<int>(crank) * q_rows_cta;
                const int sfq_g0 = (tq * bn) >> 5;
                for(int i = 0; i < n_iters; ++i, ++g)
                {
                    const int s = g % S;
                    ok = bounded_wait(empty_bar(s), ((g / S) & 1) ^ 1, abort_f, prm.status, ST_TIMEOUT_PRODUCER, g);
                    if(!ok)
                        break;
                    const uint32_t stage = smem_base + s * L.stage_bytes;
                    const uint32_t bar   = full_bar(s);
                    if(g == 5) stamp(34);
                    const bool p_f4 = kMixed && prm.f4_operand == 1, q_f4 = kMixed && prm.f4_operand == 2;
                    mbar_arrive_expect_tx(bar, (p_f4 ? kTileP * 64u : kTileP * kTileKBytes) + (q_f4 ? q_box_bytes / 2 : q_box_bytes) +
                                                   sfp_bytes + sfq_bytes);
                    if(g == 5) stamp(35);
                    // a packed e2m1 operand (always 16x16-byte tiled) lands in the staging area: 4 chunks of 16 bytes per row
                    if(p_f4)
                        tma_load_3d(stage + L.stg_off, &map_p, bar, 0, row_p0 >> 4, (it_beg + i) * 4);
                    else
                        issue_operand_load(prm.p_mode, stage, &map_p, bar, row_p0, it_beg + i);
                    if(g == 5) stamp(36);
                    if(q_f4)
                        tma_load_3d(stage + L.stg_off, &map_q, bar, 0, row_q0 >> 4, (it_beg + i) * 4);
                    else
                        issue_operand_load(prm.q_mode, stage + L.q_off, &map_q, bar, row_q0, it_beg + i);
                    if(g == 5) stamp(37);
                    if(kScaled)
                    {
                        tma_load_2d(stage + L.sfp_off, &map_sfp, bar, (it_beg + i) * kSfChunk, row_p0 >> 5);
                        if(g == 5) stamp(38);
                        tma_load_2d(stage + L.sfq_off, &map_sfq, bar, (it_beg + i) * kSfChunk, sfq_g0);
                        if(g == 5) stamp(39);
                    }
                    if(g < 8) stamp(2 + 4 * g);
                }
            }
            if(*abort_f)
            {
                // wait (bounded) for loads still in flight so that none lands after exit
                for(int j = g - 1; j >= 0 && j >= g - S; --j)
                {
                    bool done = false;
                    const uint64_t t0 = global_timer_ns();
                    while(!done && global_timer_ns() - t0 < kWaitLimitNs)
                        done = mbar_try_wait(full_bar(j % S), (j / S) & 1);
                    if(!done)
                        atomicCAS(prm.status, 0u, ST_TIMEOUT_DRAIN);
                }
            }
        }
    }
    else if(warp == 1)
    {
        if(lane == 0 && leader)
        {
            // ------------------------------------------------------------------ MMA issuer (leader CTA)
            constexpr uint32_t kM = kTileP * CG;
            uint32_t idesc;
            if(KIND == KIND_BF16)
                idesc = idesc_bf16(kM, bn);
            else if(KIND == KIND_MXF8 || KIND == KIND_MXF8F4)
                idesc = idesc_block_scaled(0, 0, kM, bn); // the e2m1 operand has been widened to e4m3 in shared memory
            else
                idesc = idesc_block_scaled(1, 1, kM, bn);
            const bool p_tiled   = (prm.p_mode == OPM_TILE16);
            const bool q_tiled   = (prm.q_mode == OPM_TILE16);
            const uint32_t p_lbo = p_tiled ? kTileP * 16u : 16u;
            const uint32_t p_sbo = p_tiled ? 128u : 1024u;
            const uint32_t p_lay = p_tiled ? 0u : 2u;
            const uint32_t p_adv = p_tiled ? 2u * kTileP * 16u : 32u;
            const uint32_t q_lbo = q_tiled ? q_rows_cta * 16u : 16u;
            const uint32_t q_sbo = q_tiled ? 128u : 1024u;
            const uint32_t q_lay = q_tiled ? 0u : 2u;
            const uint32_t q_adv = q_tiled ? 2u * q_rows_cta * 16u : 32u;

            int g = 0, uc = 0;
            bool ok = true;
            for(int u = cluster_id; u < total_units && ok; u += n_clusters, ++uc)
            {
                int tp, tq, it_beg, n_iters, z;
                decode(u, tp, tq, it_beg, n_iters, z);
                const int a          = uc % prm.n_acc;
                const uint32_t d_col = tmem_base + a * prm.acc_stride;
                ok = bounded_wait(acc_empty_bar(a), ((uc / prm.n_acc) & 1) ^ 1, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, 0x10000 + uc);
                if(!ok)
                    break;
                tc_fence_after_sync();
                for(int i = 0; i < n_iters; ++i, ++g)
                {
                    const int s          = g % S;
                    const uint32_t phase = (g / S) & 1;
                    ok = bounded_wait(full_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, g);
                    if(ok && ready_count > 0)
                        ok = bounded_wait(ready_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_MMA_SF, g);
                    if(!ok)
                        break;
                    tc_fence_after_sync();
                    if(g < 8) stamp(5 + 4 * g);
                    const uint32_t stage = smem_base + s * L.stage_bytes;
                    const uint32_t tsfp  = tmem_base + prm.sf_tmem_base + s * prm.sf_cols;
                    const uint32_t tsfq  = tsfp + sfp_cols;
#pragma unroll
                    for(int k = 0; k < 4; ++k)
                    {
                        const uint64_t pd  = make_smem_desc(stage + k * p_adv, p_lbo, p_sbo, p_lay);
                        const uint64_t qd  = make_smem_desc(stage + L.q_off + k * q_adv, q_lbo, q_sbo, q_lay);
                        const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                        if(CG == 1)
                        {
                            if(KIND == KIND_BF16)
                                mma_f16(d_col, pd, qd, idesc, acc);
                            else if(KIND == KIND_MXF8 || KIND == KIND_MXF8F4)
                                mma_mxf8f6f4(d_col, pd, qd, idesc_with_sf(idesc, k, k), acc, tsfp, tsfq);
                            else
                                mma_mxf4(d_col, pd, qd, idesc_with_sf(idesc, (k & 1) * 2, (k & 1) * 2), acc,
                                         tsfp + (k >> 1) * 4, tsfq + (k >> 1) * 4 * nq128);
                        }
                        else
                        {
                            if(KIND == KIND_BF16)
                                mma_f16_2cta(d_col, pd, qd, idesc, acc);
                            else if(KIND == KIND_MXF8 || KIND == KIND_MXF8F4)
                                mma_mxf8f6f4_2cta(d_col, pd, qd, idesc_with_sf(idesc, k, k), acc, tsfp, tsfq);
                            else
                                mma_mxf4_2cta(d_col, pd, qd, idesc_with_sf(idesc, (k & 1) * 2, (k & 1) * 2), acc,
                                              tsfp + (k >> 1) * 4, tsfq + (k >> 1) * 4 * nq128);
                        }
                    }
                    if(g == 5) stamp(42);
                    if(CG == 1)
                        tc_commit(empty_bar(s));
                    else
                        tc_commit_2cta(empty_bar(s), 3);
                    if(g == 5) stamp(43);
                }
                if(ok)
                {
                    if(CG == 1)
                        tc_commit(acc_full_bar(a));
                    else
                        tc_commit_2cta(acc_full_bar(a), 3);
                }
            }
            stamp(60);
            if(!ok)
            {
                // abort: let whatever was issued finish before TMEM is released
                if(CG == 1)
                    tc_commit(drain_bar);
                else
                    tc_commit_2cta(drain_bar, 1);
                const uint64_t t0 = global_timer_ns();
                while(!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < kWaitLimitNs) {}
            }
        }
        else if(lane == 0 && CG == 2 && !kScaled)
        {
            // ------------------------------------------------------------------ second CTA of a bf16 pair:
            // tell the leader when this CTA's half of a stage has landed
            int g = 0;
            bool ok = true;
            for(int u = cluster_id; u < total_units && ok; u += n_clusters)
            {
                int tp, tq, it_beg, n_iters, z;
                decode(u, tp, tq, it_beg, n_iters, z);
                for(int i = 0; i < n_iters; ++i, ++g)
                {
                    const int s = g % S;
                    ok = bounded_wait(full_bar(s), (g / S) & 1, abort_f, prm.status, ST_TIMEOUT_SFWARP, g);
                    if(!ok)
                        break;
                    mbar_arrive_cluster(map_to_cta(ready_bar(s), 0));
                }
            }
        }
    }
    else if(warp < 6)
    {
        // ------------------------------------------------------------------ scale warps (every CTA)
        if(kScaled)
        {
            const int quarter    = warp & 3;
            const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            const uint32_t ready_remote = (CG == 2) ? map_to_cta(ready_bar(0), 0) : 0u;
            int g = 0;
            bool ok = true;
            for(int u = cluster_id; u < total_units && ok; u += n_clusters)
            {
                int tp, tq, it_beg, n_iters, z;
                decode(u, tp, tq, it_beg, n_iters, z);
                for(int i = 0; i < n_iters; ++i, ++g)
                {
                    const int s = g % S;
                    ok = bounded_wait(full_bar(s), (g / S) & 1, abort_f, prm.status, ST_TIMEOUT_SFWARP, g);
                    ok = __all_sync(0xffffffffu, ok);
                    if(!ok)
                        break;
                    if(warp == 2 && lane == 0 && g < 8) stamp(3 + 4 * g);
                    uint8_t* stage = smem_gen + s * L.stage_bytes;
                    const uint32_t tsfp  = tlane + prm.sf_tmem_base + s * prm.sf_cols;
                    const uint32_t tsfq  = tsfp + sfp_cols;
                    if(kMixed)
                    {
                        // widen the packed e2m1 operand of this stage to e4m3 in the MMA's un-swizzled layout:
                        // staging [4 chunks][rows][16 B] (32 codes) -> tile [8 chunks][rows][16 B]
                        const int rows     = (prm.f4_operand == 1) ? kTileP : q_rows_cta;
                        const uint4* src   = reinterpret_cast<const uint4*>(stage + L.stg_off);
                        uint4* dst         = reinterpret_cast<uint4*>(stage + (prm.f4_operand == 1 ? 0u : L.q_off));
                        const int items    = rows * 4;
                        for(int it = (warp - 2) * 32 + lane; it < items; it += 128)
                        {
                            const int kc  = it / rows;
                            const int r   = it - kc * rows;
                            const uint4 v = src[it];
                            uint4 o0, o1;
                            e2m1x8_to_e4m3x8(v.x, o0.x, o0.y);
                            e2m1x8_to_e4m3x8(v.y, o0.z, o0.w);
                            e2m1x8_to_e4m3x8(v.z, o1.x, o1.y);
                            e2m1x8_to_e4m3x8(v.w, o1.z, o1.w);
                            dst[(2 * kc) * rows + r]     = o0;
                            dst[(2 * kc + 1) * rows + r] = o1;
                        }
                        fence_proxy_async_smem(); // these generic-proxy writes are read by the tensor core
                    }
                    for(int op = 0; op < 2; ++op)
                    {
                        const uint32_t* region = reinterpret_cast<const uint32_t*>(stage + (op == 0 ? L.sfp_off : L.sfq_off));
                        const int groups       = (op == 0) ? prm.sf_groups_p : prm.sf_groups_q;
                        const int blocks       = (op == 0) ? 1 : nq128;
                        const uint32_t tbase   = (op == 0) ? tsfp : tsfq;
                        if(SFW == SFW_G1250)
                        {
                            // wire: [group][k quarter a][row 0..31][4 k-blocks]
                            for(int nb = 0; nb < blocks; ++nb)
#pragma unroll
                                for(int a = 0; a < kAtomsK; ++a)
                                {
                                    uint32_t w[4];
#pragma unroll
                                    for(int g4 = 0; g4 < 4; ++g4)
                                    {
                                        const int gg = nb * 4 + g4;
                                        w[g4]        = (gg < groups) ? region[gg * (32 * kAtomsK) + a * 32 + lane] : 0x7F7F7F7Fu;
                                    }
                                    tmem_st_x4(tbase + (a * blocks + nb) * 4, w[0], w[1], w[2], w[3]);
                                }
                        }
                        else if(SFW == SFW_E8M0_SHUFFLE)
                        {
                            // wire: per 32-row group and 8 k-blocks a 256-byte chunk, byte offset
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
                                        const int gg = nb * 4 + g4;
                                        w[g4][kk]    = (gg < groups) ? region[gg * 64 + kk * 16 + r16] : 0x7F7F7F7Fu;
                                    }
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
                                    tmem_st_x4(tbase + (kh * blocks + nb) * 4, o[0], o[1], o[2], o[3]);
                                }
                            }
                        }
                    }
                    if(warp == 2 && lane == 0 && g == 5) stamp(40);
                    tmem_st_wait();
                    if(warp == 2 && lane == 0 && g == 5) stamp(41);
                    tc_fence_before_sync();
                    __syncwarp();
                    if(lane == 0)
                    {
                        if(CG == 2)
                            mbar_arrive_cluster(ready_remote + 8u * s);
                        else
                            mbar_arrive(ready_bar(s));
                        if(warp == 2 && g < 8) stamp(4 + 4 * g);
                    }
                }
            }
        }
    }
    else
    {
        // ------------------------------------------------------------------ epilogue (warps 6..9, every CTA)
        const int quarter    = warp & 3;
        const int p_local    = quarter * 32 + lane;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const int chunk      = bn < 32 ? 16 : 32;
        const int n_chunks   = bn / chunk;
        const bool split     = (splits > 1);
        const uint32_t acc_empty_remote = (CG == 2) ? map_to_cta(acc_empty_bar(0), 0) : 0u;
        const bool vec_ok = (!prm.transposed_out) && ((prm.ldo & 7) == 0) && ((reinterpret_cast<uintptr_t>(prm.out) & 15) == 0);
        uint32_t epi_phase = 0;
        int uc = 0;
        bool ok = true;
        for(int u = cluster_id; u < total_units && ok; u += n_clusters, ++uc)
        {
            int tp, tq, it_beg, n_iters, z;
            decode(u, tp, tq, it_beg, n_iters, z);
            const int a       = uc % prm.n_acc;
            const int p       = (tp * CG + static_cast<int>(crank)) * kTileP + p_local;
            const int row_q0  = tq * bn;
            const int slot    = (tp * prm.tiles_q + tq) * CG + static_cast<int>(crank); // one ticket / partial slot per CTA tile
            ok = bounded_wait(acc_full_bar(a), (uc / prm.n_acc) & 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, uc);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                break;
            tc_fence_after_sync();
            if(warp == 6 && lane == 0 && uc == 0) stamp(61);
            const uint32_t tacc = tlane + a * prm.acc_stride;
            bool is_last        = !split;

            if(split)
            {
                float* mine = prm.ws_partial + (static_cast<size_t>(slot) * splits + z) * (static_cast<size_t>(bn) * kTileP);
                for(int c = 0; c < n_chunks; ++c)
                {
                    uint32_t r[32];
                    if(chunk == 32)
                        tmem_ld_x32(tacc + c * 32, r);
                    else
                        tmem_ld_x16(tacc + c * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                        if(j < chunk)
                            mine[static_cast<size_t>(c * chunk + j) * kTileP + p_local] = __uint_as_float(r[j]);
                }
                // the accumulator is drained: hand it back before the reduction
                tc_fence_before_sync();
                __syncwarp();
                if(lane == 0)
                {
                    if(CG == 2)
                        mbar_arrive_cluster(acc_empty_remote + 8u * a);
                    else
                        mbar_arrive(acc_empty_bar(a));
                }
                __threadfence();
                __syncwarp();
                if(lane == 0)
                    mbar_arrive(epi_bar);
                ok = bounded_wait(epi_bar, epi_phase, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x1000 + uc);
                ok = __all_sync(0xffffffffu, ok);
                epi_phase ^= 1;
                if(ok)
                {
                    if(warp == 6 && lane == 0)
                    {
                        *reinterpret_cast<volatile uint32_t*>(ticket_smem) = atomicAdd(prm.ws_counter + slot, 1u);
                        __threadfence_block();
                    }
                    __syncwarp();
                    if(lane == 0)
                        mbar_arrive(epi_bar);
                    ok = bounded_wait(epi_bar, epi_phase, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x2000 + uc);
                    ok = __all_sync(0xffffffffu, ok);
                    epi_phase ^= 1;
                }
                if(!ok)
                    break;
                is_last = (*reinterpret_cast<volatile uint32_t*>(ticket_smem) == static_cast<uint32_t>(splits - 1));
                if(is_last)
                    __threadfence();
            }

            if(is_last)
            {
                const float* part = split ? prm.ws_partial + static_cast<size_t>(slot) * splits * (static_cast<size_t>(bn) * kTileP) : nullptr;
                for(int c = 0; c < n_chunks; ++c)
                {
                    float v[32];
                    if(!split)
                    {
                        uint32_t r[32];
                        if(chunk == 32)
                            tmem_ld_x32(tacc + c * 32, r);
                        else
                            tmem_ld_x16(tacc + c * 16, r);
                        tmem_ld_wait();
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                            v[j] = __uint_as_float(r[j]);
                        if(c == n_chunks - 1)
                        {
                            // every column of this accumulator is in registers now: hand it back
                            tc_fence_before_sync();
                            __syncwarp();
                            if(lane == 0)
                            {
                                if(CG == 2)
                                    mbar_arrive_cluster(acc_empty_remote + 8u * a);
                                else
                                    mbar_arrive(acc_empty_bar(a));
                            }
                        }
                    }
                    else
                    {
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                            v[j] = 0.f;
                        for(int zz = 0; zz < splits; ++zz)
                        {
                            const float* src = part + static_cast<size_t>(zz) * (static_cast<size_t>(bn) * kTileP);
#pragma unroll
                            for(int j = 0; j < 32; ++j)
                                if(j < chunk)
                                    v[j] += __ldcg(src + static_cast<size_t>(c * chunk + j) * kTileP + p_local);
                        }
                    }
                    const int q_first = row_q0 + c * chunk;
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
                                        *reinterpret_cast<uint4*>(dst + j) =
                                            make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                                                       pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
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
                if(split && warp == 6 && lane == 0)
                    prm.ws_counter[slot] = 0; // ready for the next launch
            }
            else if(!split)
            {
                // unreachable: without split-K every unit is final
            }
        }
        if(warp == 6 && lane == 0) stamp(62);
        tc_fence_before_sync();
    }

    __syncthreads();
    if(CG == 2)
        cluster_sync_all(); // nobody leaves while the partner may still arrive on this CTA's barriers
    if(threadIdx.x == 0) stamp(63);
    if(warp == 1)
    {
        tc_fence_after_sync();
        if(CG == 2)
            tmem_dealloc_2cta(tmem_base, static_cast<uint32_t>(prm.tmem_cols));
        else
            tmem_dealloc(tmem_base, static_cast<uint32_t>(prm.tmem_cols));
    }
}

} // namespace b200
