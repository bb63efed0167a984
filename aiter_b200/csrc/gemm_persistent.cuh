// Persistent warp-specialised tcgen05 GEMM for sm_100a, optionally on CTA pairs (cta_group::2).
//
//   D[p][q] = sum_k P[p][k] * Q[q][k]      P: 128 rows per CTA on the TMEM lanes, Q: BN columns
//
// One CTA (CG = 1) or one pair of CTAs on neighbouring SMs (CG = 2) walks a static list of work units
// (output tile x K split).  In a pair every CTA stages its own 128 rows of P and its own half of the BN
// rows of Q; the leader's MMA thread issues 256 x BN instructions that read both CTAs' shared memory, so
// each SM moves 2/3 of the bytes per flop of the single-CTA tile (the fill rate of shared memory, 64 B per
// clock per SM, is what bounds these kernels).  No TMA multicast is used anywhere: every CTA fetches
// exactly the bytes it stages.
//
// Warps (384 threads per CTA):
//   0, 10  TMA producers for the P and the Q operand tiles (one thread each: issuing a 16 KB tile load keeps
//          a thread busy for a few hundred cycles, so the two operands are issued in parallel); completion
//          bytes of BOTH CTAs of a pair are counted on the leader's barrier
//   11     TMA producer for the raw UE8M0 block scales (wire layout) of each stage
//   1      MMA issuer (leader CTA) and TMEM owner
//   2..5   scale warps, one per TMEM lane quarter: read a stage's raw scale bytes from shared memory in
//          whatever wire layout the caller uses, re-order them in registers and write them to a per-stage
//          TMEM buffer with tcgen05.st.  For the mixed e4m3 x e2m1 kind they also widen the packed e2m1
//          operand to e4m3 in shared memory.
//   6..9   epilogue: TMEM -> registers -> alpha/bias -> bf16 -> global (or split-K partials + last-arriver
//          reduction), overlapped with the next unit's main loop when two accumulators fit in TMEM
//
// Barriers (all waits bounded by wall time):
//   full[s]       leader: the operand tiles of stage s of every CTA of the pair have landed and every scale warp
//                 of every CTA has written the stage's scales to TMEM (one wait for the MMA issuer)
//   staged[s]     mixed kind: this CTA's packed e2m1 tile of stage s has landed (local)
//   sfraw[s]      this CTA's raw scale bytes of stage s have landed (local)
//   xch[s]        e8m0_shuffle wire layout: the four scale warps have re-ordered their share of stage s (local)
//   empty[s]      the MMAs reading stage s (and its TMEM scales) are done (tcgen05.commit, both CTAs)
//   acc_full[a]   accumulator a is complete (tcgen05.commit, both CTAs)
//   acc_empty[a]  leader: all epilogue warps of all CTAs have drained accumulator a
#pragma once
#include "gemm_common.cuh"

namespace b200 {

constexpr int kPersistentThreads = 384;
constexpr int kMaxAcc            = 2;

struct PersistentParams
{
    int rows_p, rows_q;
    int num_k_iters;  // ceil(K elements / elements per 128-byte tile)
    int kblocks;      // valid 32-element scale blocks along K
    int bn;           // UMMA N (multiple of 16, <= 256; multiple of 32 unless there is a single Q tile)
    int stages;
    int p_mode, q_mode;
    int f4_operand;   // mixed kind only: which operand arrives as packed e2m1 (1 = P, 2 = Q)
    int transposed_out;
    int tiles_p, tiles_q, splits; // tiles_p counts 128*CG-row tiles
    int n_acc;                    // accumulators in TMEM (1 or 2)
    int acc_stride;               // TMEM columns between accumulators
    int sf_tmem_base;             // first TMEM column of the per-stage scale buffers
    int sf_cols;                  // TMEM columns per stage for scales
    int csplit;                   // K split across the CTAs of a thread-block cluster (1 = none; CG == 1 only, one tile per cluster)
    int split_shift;              // log2 of the K split in use (csplit if > 1, else splits) when it is a power of two, else -1
    int tma_store;                // the output goes through shared memory and TMA tile stores (map_out is valid)
    int epi_bufs;                 // staging areas reserved for that: 0 none, 1, or 2 (wide stores double-buffered)
    int panel_q;                  // tile order: Q tiles per L2-sized panel (0: Q fastest over the whole width)
    int tmem_cols;                // allocation (power of two)
    // block scales in global memory (wire layout), one "group" = 32 rows; a group row is `sf_row_words` words
    const uint32_t* sfp;
    const uint32_t* sfq;
    int sfp_groups, sfq_groups;   // groups present in each scale tensor
    int sfp_row_words, sfq_row_words;
    void* out;                    // bf16 / fp16 / fp32 [M][N], packed e2m1 [M][N/2] or e4m3 [M][N] (see out_mode)
    long long ldo;                // row pitch in output elements (bytes for the e2m1 / e4m3 outputs)
    int out_mode;                 // OutMode
    uint8_t* out_scale;           // OUT_MXFP8: UE8M0 per (row, 128 columns) in the packed (M/64, N/128, 16, 4) byte order
    int out_scale_cols;           // N / 128
    int noscale;                  // the block scales are not applied (every scale byte reads 2^0): the reference's fp4-output GEMM
    int batch;                    // batched problem: number of [M,K] x [N,K] pairs (1: plain); tiles_p counts one pair's tiles
    long long out_batch_stride;   // output elements between two pairs' outputs
    long long bias_batch_stride;  // bias elements between two pairs' bias vectors (0: shared)
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
    uint32_t stage_bytes, q_off, sfp_off, sfq_off, stg_off, epi_off, red_off, bar_off, total;
};

constexpr uint32_t kEpiStageBytes = 16384; // 4 epilogue warps x 4 KB: two 32 x 64-byte buffers, or one 32 x 128-byte buffer (wide
                                           // stores); twice that when the wide stores are double-buffered

// scaled: 0 no scales; 1 the stage carries 1 KB + 2 KB of raw scale bytes (P groups, Q groups: 256 bytes per group of 32
//         rows); 2 twice that (NVFP4: 512 bytes per group) - sf_unit_of(kind)
// f4_operand: 0 none, 1 = P, 2 = Q arrives as packed e2m1 and needs a staging area of rows x 64 bytes
// epi_stage: 0 none, 1 the epilogue's output staging area (tile stores through TMA), 2 twice the area
// csplit: cluster K split; its leader keeps (csplit - 1) partial tiles of 128 x bn floats
__host__ __device__ inline PersistentSmem make_persistent_smem(int bn, int cg, int stages, int f4_operand, int scaled,
                                                               int epi_stage, int csplit)
{
    PersistentSmem L;
    uint32_t q_bytes = static_cast<uint32_t>(bn / cg) * kTileKBytes;
    q_bytes          = (q_bytes + 1023u) & ~1023u;
    L.q_off          = kTileP * kTileKBytes;
    L.sfp_off        = L.q_off + q_bytes;
    L.sfq_off        = L.sfp_off + 1024u * static_cast<uint32_t>(scaled);
    L.stg_off        = L.sfq_off + 2048u * static_cast<uint32_t>(scaled);
    uint32_t stg     = f4_operand == 1 ? kTileP * 64u : (f4_operand == 2 ? static_cast<uint32_t>(bn / cg) * 64u : 0u);
    stg              = (stg + 1023u) & ~1023u;
    L.stage_bytes    = L.stg_off + stg;
    L.epi_off        = L.stage_bytes * static_cast<uint32_t>(stages);
    L.red_off        = L.epi_off + static_cast<uint32_t>(epi_stage) * kEpiStageBytes;
    // up to four slices: every CTA receives the other slices' share of its own 128 / csplit rows; eight: the first CTA all
    const uint32_t red_rows = csplit <= 1 ? 0u : static_cast<uint32_t>(csplit - 1) * (csplit <= 4 ? static_cast<uint32_t>(kTileP / csplit) : static_cast<uint32_t>(kTileP));
    L.bar_off        = L.red_off + red_rows * static_cast<uint32_t>(bn) * 4u;
    L.total          = L.bar_off + 512u;
    return L;
}

// TMEM columns one stage's scales occupy: [P atoms: 4 per K atom][Q atoms: 8 per K atom (two 128-row blocks)]
__host__ __device__ constexpr int sf_cols_per_stage(int kind)
{
    return kind == KIND_BF16 ? 0 : (kind == KIND_NVF4 ? 48 : (kind == KIND_MXF4 ? 24 : 16));
}
// raw scale bytes of a stage in units of 256 per 32-row group (the `scaled` argument of make_persistent_smem)
__host__ __device__ constexpr int sf_unit_of(int kind) { return kind == KIND_BF16 ? 0 : (kind == KIND_NVF4 ? 2 : 1); }

// Stage ring position kept by increments: these loops run on one thread (or one warp) per K tile, where a
// division by the run-time stage count would cost more than the work itself.
struct Ring
{
    int s;
    uint32_t phase;
    __device__ __forceinline__ void advance(int stages)
    {
        if(++s == stages)
        {
            s = 0;
            phase ^= 1u;
        }
    }
};

// Position in the static work list shared by all roles of a CTA.
struct WorkIter
{
    int u, i, tp, tq, it_beg, n_iters, z, b; // b: pair of a batched problem
    bool valid;
};

template <int KIND, int SFW, int CG>
__global__ void __launch_bounds__(kPersistentThreads, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_sfp, const __grid_constant__ CUtensorMap map_sfq,
                       const __grid_constant__ CUtensorMap map_out, const PersistentParams prm)
{
    constexpr bool kScaled = (KIND != KIND_BF16);
    constexpr bool kMixed  = (KIND == KIND_MXF8F4);
    constexpr bool kNvf4   = (KIND == KIND_NVF4);
    // scale atoms per 128-byte K tile: one 32-bit word per row each (MX: the scales of 4 blocks of 32; NVFP4: of 4 blocks of 16)
    constexpr int kAtomsK  = kNvf4 ? 4 : ((KIND == KIND_MXF4) ? 2 : 1);
    constexpr int kSfCols  = sf_cols_per_stage(KIND);
    constexpr int kTWords  = kSfCols > 24 ? 48 : (kSfCols > 16 ? 24 : 16);
    constexpr uint32_t kNeutralSf = kNvf4 ? 0x38383838u : 0x7F7F7F7Fu; // four scale bytes of 1.0 (e4m3 / e8m0)

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen        = smem_raw + (smem_base - smem_u32(smem_raw));
    const int bn             = prm.bn;
    const int S              = prm.stages;
    const PersistentSmem L   = make_persistent_smem(bn, CG, S, kMixed ? prm.f4_operand : 0, sf_unit_of(KIND), prm.epi_bufs, prm.csplit);
    constexpr int kSfChunk   = (SFW == SFW_E8M0_SHUFFLE) ? 256 : 128 * kAtomsK; // raw scale bytes per 32-row group per stage

    const uint32_t bar_base  = smem_base + L.bar_off;
    auto full_bar            = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar           = [&](int s) { return bar_base + 128u + 8u * s; };
    auto staged_bar          = [&](int s) { return bar_base + 192u + 8u * s; };
    auto sfraw_bar           = [&](int s) { return bar_base + 256u + 8u * s; };
    auto xch_bar             = [&](int s) { return bar_base + 320u + 8u * s; };
    auto acc_full_bar        = [&](int a) { return bar_base + 384u + 8u * a; };
    auto acc_empty_bar       = [&](int a) { return bar_base + 400u + 8u * a; };
    const uint32_t epi_bar   = bar_base + 416u;
    const uint32_t drain_bar = bar_base + 424u;
    const uint32_t red_bar   = bar_base + 448u;
    uint32_t* tmem_ptr_smem    = reinterpret_cast<uint32_t*>(smem_gen + L.bar_off + 432);
    volatile uint32_t* abort_f = reinterpret_cast<volatile uint32_t*>(smem_gen + L.bar_off + 436);
    uint32_t* ticket_smem      = reinterpret_cast<uint32_t*>(smem_gen + L.bar_off + 440);

    const int warp       = threadIdx.x >> 5;
    const int lane       = threadIdx.x & 31;
    const int csplit        = (CG == 1) ? prm.csplit : 1;
    const uint32_t hw_rank  = (CG == 2 || csplit > 1) ? cluster_ctarank() : 0u;
    const uint32_t crank    = (CG == 2) ? hw_rank : 0u; // 0 = leader of a CTA pair
    const uint32_t zrank    = (csplit > 1) ? hw_rank : 0u; // K slice of a cluster-split tile; 0 = the reducing CTA
    const bool leader       = (crank == 0);
    const int cluster_ctas  = CG * csplit;
    const int cluster_id    = blockIdx.x / cluster_ctas;
    const int n_clusters    = gridDim.x / cluster_ctas;

    B200_TRACE(const bool tracing = (prm.trace != nullptr) && blockIdx.x == 0;)
    B200_TRACE(auto stamp = [&](int slot) { if(tracing && slot < 64) prm.trace[slot] = static_cast<unsigned long long>(clock64()); };)
    B200_TRACE(if(threadIdx.x == 0) stamp(0);)
    B200_TRACE(if(prm.trace != nullptr && threadIdx.x == 0 && blockIdx.x < 160) prm.trace[64 + 2 * blockIdx.x] = global_timer_ns();)

    const int splits      = prm.splits;
    const int total_units = prm.batch * prm.tiles_p * prm.tiles_q * (prm.csplit > 1 ? 1 : splits);

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < S; ++s)
        {
            // one expect_tx arrival per operand producer and one arrival per scale warp, of every CTA of the pair
            // producers + scale warps (+ widening warps: all four of them, or one pair of them on a 128-row packed tile)
            mbar_init(full_bar(s), (kMixed ? ((prm.f4_operand == 1 || prm.bn / CG == kTileP) ? 8 : 10) : (kScaled ? 6 : 2)) * CG);
            mbar_init(empty_bar(s), 1);
            mbar_init(staged_bar(s), 1);
            mbar_init(sfraw_bar(s), kMixed ? 2 : 1); // raw scales (+ the packed e2m1 tile of the mixed kind: one wait covers both)
            mbar_init(xch_bar(s), 4);
        }
        for(int a = 0; a < kMaxAcc; ++a)
        {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 4 * CG);
        }
        mbar_init(epi_bar, 4);
        mbar_init(drain_bar, 1);
        mbar_init(red_bar, 1);
        *abort_f = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
        B200_TRACE(stamp(40);)
    }
    if(warp == 10 && lane == 0)
    {
        // the descriptor fetch (about a microsecond, cold) runs while thread 0 initialises the barriers
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
    B200_TRACE(if(threadIdx.x == 0) stamp(41);)
    if(CG == 2)
        cluster_sync_all(); // the partner's barriers exist before anything arrives on them remotely
    else if(csplit > 1)
        cluster_arrive_release(); // K-split cluster: announced here, checked by the epilogue before its first remote access
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    B200_TRACE(if(threadIdx.x == 0) stamp(1);)
    // Programmatic dependent launch: everything above (barriers, TMEM, descriptor prefetch) may overlap the tail of
    // the previous kernel in the stream; nothing below may touch global memory before that kernel has completed.
    // The next kernel's CTAs may in turn be scheduled as soon as every CTA of this grid has got here.
    grid_dependency_wait();
    grid_launch_dependents();
    B200_TRACE(if(threadIdx.x == 0) stamp(42);)

    const int q_rows_cta       = bn / CG;
    const uint32_t q_box_bytes = static_cast<uint32_t>(q_rows_cta) * kTileKBytes;
    const int nq128            = (bn + 127) / 128;
    const bool p_f4            = kMixed && prm.f4_operand == 1;
    const bool q_f4            = kMixed && prm.f4_operand == 2;

    // unit -> (tile_p, tile_q, k range); q runs fastest so that concurrently running CTAs share P tiles
    auto decode = [&](WorkIter& w) {
        w.valid = w.u < total_units;
        if(!w.valid)
            return;
        // Every role decodes its first unit before it can start, one thread paying each instruction's latency: the
        // usual cases (power-of-two K split, a single Q tile) take shifts instead of ~150-cycle integer divisions.
        const int ksplit = (csplit > 1) ? csplit : splits;
        const int sh     = prm.split_shift;
        int tile;
        if(csplit > 1)
        {
            w.z  = static_cast<int>(zrank);
            tile = w.u;
        }
        else if(sh >= 0)
        {
            w.z  = w.u & (splits - 1);
            tile = w.u >> sh;
        }
        else
        {
            w.z  = w.u % splits;
            tile = w.u / splits;
        }
        w.b = 0;
        if(prm.batch > 1)
        {
            const int per_pair = prm.tiles_p * prm.tiles_q;
            w.b                = tile / per_pair;
            tile -= w.b * per_pair;
        }
        if(prm.tiles_q == 1)
        {
            w.tq = 0;
            w.tp = tile;
        }
        else if(prm.panel_q > 0)
        {
            // L2-sized panels of the Q operand: all P tiles against panel 0's Q tiles (Q fastest inside the panel), then
            // panel 1, ...  The panel's Q rows stay in L2 while P streams past once per panel; without panels a Q operand
            // larger than L2 is read from HBM once per row of tiles.
            const int panel_tiles = prm.tiles_p * prm.panel_q; // every panel but the last is this large
            const int pn          = tile / panel_tiles;
            const int r           = tile - pn * panel_tiles;
            const int q0          = pn * prm.panel_q;
            const int wq          = min(prm.panel_q, prm.tiles_q - q0);
            w.tp                  = r / wq;
            w.tq                  = q0 + (r - w.tp * wq);
        }
        else
        {
            w.tq = tile % prm.tiles_q;
            w.tp = tile / prm.tiles_q;
        }
        // num_k_iters * splits < 2^31 (checked on the host)
        if(sh >= 0)
        {
            w.it_beg  = (prm.num_k_iters * w.z) >> sh;
            w.n_iters = ((prm.num_k_iters * (w.z + 1)) >> sh) - w.it_beg;
        }
        else
        {
            w.it_beg  = static_cast<int>(static_cast<uint32_t>(prm.num_k_iters * w.z) / static_cast<uint32_t>(ksplit));
            w.n_iters = static_cast<int>(static_cast<uint32_t>(prm.num_k_iters * (w.z + 1)) / static_cast<uint32_t>(ksplit)) - w.it_beg;
        }
        w.i            = 0;
    };
    auto first_work = [&]() {
        WorkIter w;
        w.u = cluster_id;
        decode(w);
        return w;
    };
    auto next_unit = [&](WorkIter& w) {
        w.u += n_clusters;
        decode(w);
    };
    auto next_iter = [&](WorkIter& w) {
        if(++w.i == w.n_iters)
            next_unit(w);
    };

    // ------------------------------------------------------------------ one K tile's block scales
    // Raw scale bytes of stage s (whatever wire layout the caller uses) -> registers -> the stage's TMEM scale buffer,
    // then this warp's arrival on full[s].  Run by the four scale warps, one per TMEM lane quarter, once per K tile, so
    // it is kept short: a handful of shared-memory loads, a few byte permutes, one tcgen05.st.  (Letting the four
    // epilogue warps take every other K tile of decode shapes was measured: slower for short K, 4 % faster at K = 16384.)
    constexpr bool kE8 = (SFW == SFW_E8M0_SHUFFLE);
    auto scale_tile = [&](const int s, const uint32_t phase, const int kt, const int g) -> bool {
        const int quarter    = warp & 3;
        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t full_leader = (CG == 2) ? map_to_cta(full_bar(0), 0) : full_bar(0);
        const int r16 = lane & 15, hi = lane >> 4;
        const int q_groups = (bn + 31) / 32; // 32-row groups of Q staged per stage (P always stages 4)
        // raw scales of stage s have landed (their producer waited for the previous pass's MMAs, so the
        // TMEM scale buffer of stage s is free as well); mixed kind: the packed e2m1 tile counts on the same barrier
        bool ok = bounded_wait(sfraw_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_SFWARP, g);
        const bool widen_here = kMixed && (p_f4 || q_rows_cta == kTileP); // 128-row packed tile: k chunk 3 is ours
        ok = __all_sync(0xffffffffu, ok);
        if(!ok)
            return false;
        B200_TRACE(if(tracing && warp == 2 && lane == 0 && g < 8) stamp(3 + 4 * g);)
        uint8_t* stage = smem_gen + s * L.stage_bytes;
        if(widen_here)
        {
            const int tid = (warp - 2) * 32 + lane;
            const uint4 v = reinterpret_cast<const uint4*>(stage + L.stg_off)[3 * kTileP + tid];
            uint4* dst    = reinterpret_cast<uint4*>(stage + (p_f4 ? 0u : L.q_off));
            uint4 o0, o1;
            e2m1x8_to_e4m3x8(v.x, o0.x, o0.y);
            e2m1x8_to_e4m3x8(v.y, o0.z, o0.w);
            e2m1x8_to_e4m3x8(v.z, o1.x, o1.y);
            e2m1x8_to_e4m3x8(v.w, o1.z, o1.w);
            dst[6 * kTileP + tid] = o0;
            dst[7 * kTileP + tid] = o1;
            fence_proxy_async_smem(); // read by the tensor core
        }
        // TMEM words of this stage, column order [P atom a][Q atom a, block 0][Q atom a, block 1]
        const uint32_t* rawp = reinterpret_cast<const uint32_t*>(stage + L.sfp_off);
        const uint32_t* rawq = reinterpret_cast<const uint32_t*>(stage + L.sfq_off);
            uint32_t t[kTWords];
#pragma unroll
        for(int c = 0; c < kTWords; ++c)
            t[c] = kNeutralSf;
        if(prm.noscale)
        {
            // every scale reads 2^0: the raw bytes are loaded (the barrier protocol stays the same) and ignored
        }
        else if(kE8 && q_groups <= 2)
        {
            // Decode tiles (at most 64 rows on the Q side: six groups in all): every warp re-orders all six
            // chunks itself.  That is 24 shared-memory loads and as many byte permutes per K tile, but no
            // write-back, no rendezvous with the other three warps and no second round of loads, which at a
            // lone warp's instruction latency cost more than the re-ordering they share.
            const uint32_t* chunks = reinterpret_cast<const uint32_t*>(stage + L.sfp_off); // P's 4 chunks, then Q's
            const bool tail        = (kt * 8 + 8 > prm.kblocks);
            const uint32_t sel     = hi ? 0x7351u : 0x6240u; // bytes {kh=0, kh=1} of this lane's row half
            uint32_t raw[6][4];
#pragma unroll
            for(int j = 0; j < 6; ++j)
#pragma unroll
                for(int c = 0; c < 4; ++c)
                    raw[j][c] = (j < 4 + q_groups) ? chunks[j * 64 + c * 16 + r16] : 0u;
#pragma unroll
            for(int j = 0; j < 6; ++j)
            {
                const uint32_t lo_part = __byte_perm(raw[j][0], raw[j][1], sel); // k%4 = 0,1 for both k halves
                const uint32_t hi_part = __byte_perm(raw[j][2], raw[j][3], sel); // k%4 = 2,3
                uint32_t v0 = __byte_perm(lo_part, hi_part, 0x5410);             // k-blocks 0..3 of this row
                uint32_t v1 = __byte_perm(lo_part, hi_part, 0x7632);             // k-blocks 4..7
                if(tail)
                {
                    const int valid0  = min(max(prm.kblocks - kt * 8, 0), 4);
                    const int valid1  = min(max(prm.kblocks - kt * 8 - 4, 0), 4);
                    const uint32_t m0 = valid0 >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid0)) - 1u);
                    const uint32_t m1 = valid1 >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid1)) - 1u);
                    v0 = (v0 & m0) | (0x7F7F7F7Fu & ~m0);
                    v1 = (v1 & m1) | (0x7F7F7F7Fu & ~m1);
                }
                if(j < 4 + q_groups)
                {
                    t[(j < 4) ? j : 8 + (j - 4)]      = v0; // K atom 0: P cols 0..3, Q cols 8..
                    t[(j < 4) ? 4 + j : 16 + (j - 4)] = v1; // K atom 1: P cols 4..7, Q cols 16..
                }
            }
        }
        else if(kE8)
        {
            // raw: per 32-row group j a 256-byte chunk, byte (k%4)*64 + (m%16)*4 + ((k%8)/4)*2 + (m%32)/16:
            // word column kk = k%4, byte kh*2 + mh (mh = this lane's row half).  The re-ordering is the
            // same for all four TMEM lane quarters, so the warps share it: warp q re-orders groups q, q+4
            // and q+8 and writes the two result words per row back over the chunk it just read
            // ([k half][row 0..31]); after a (bounded) rendezvous every warp reads all 24 columns.
            uint32_t* chunks = reinterpret_cast<uint32_t*>(stage + L.sfp_off); // 12 chunks, P's 4 then Q's 8
            const bool tail  = (kt * 8 + 8 > prm.kblocks);
            uint32_t v0[3], v1[3];
#pragma unroll
            for(int jj = 0; jj < 3; ++jj)
            {
                const int j         = (warp - 2) + 4 * jj;
                const uint32_t* grp = chunks + j * 64;
                const uint32_t w0 = grp[r16], w1 = grp[16 + r16], w2 = grp[32 + r16], w3 = grp[48 + r16];
                const uint32_t sel     = hi ? 0x7351u : 0x6240u; // bytes {kh=0, kh=1} of this lane's row half
                const uint32_t lo_part = __byte_perm(w0, w1, sel); // k%4 = 0,1 for both k halves
                const uint32_t hi_part = __byte_perm(w2, w3, sel); // k%4 = 2,3
                v0[jj] = __byte_perm(lo_part, hi_part, 0x5410); // k-blocks 0..3 of this row
                v1[jj] = __byte_perm(lo_part, hi_part, 0x7632); // k-blocks 4..7
                if(tail)
                {
                    const int valid0  = min(max(prm.kblocks - kt * 8, 0), 4);
                    const int valid1  = min(max(prm.kblocks - kt * 8 - 4, 0), 4);
                    const uint32_t m0 = valid0 >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid0)) - 1u);
                    const uint32_t m1 = valid1 >= 4 ? 0xFFFFFFFFu : ((1u << (8 * valid1)) - 1u);
                    v0[jj] = (v0[jj] & m0) | (0x7F7F7F7Fu & ~m0);
                    v1[jj] = (v1[jj] & m1) | (0x7F7F7F7Fu & ~m1);
                }
                const bool in = (j < 4) || (j - 4 < q_groups);
                if(!in)
                    v0[jj] = v1[jj] = 0x7F7F7F7Fu;
            }
            __syncwarp(); // every lane has read this warp's chunks
#pragma unroll
            for(int jj = 0; jj < 3; ++jj)
            {
                uint32_t* grp = chunks + ((warp - 2) + 4 * jj) * 64;
                grp[lane]      = v0[jj];
                grp[32 + lane] = v1[jj];
            }
            __syncwarp();
            if(lane == 0)
                mbar_arrive(xch_bar(s));
            ok = bounded_wait(xch_bar(s), phase, abort_f, prm.status, ST_TIMEOUT_SFWARP, 0x30000 + g);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                return false;
#pragma unroll
            for(int j = 0; j < 12; ++j)
            {
                t[(j < 4) ? j : 8 + (j - 4)]      = chunks[j * 64 + lane];      // K atom 0: P cols 0..3, Q cols 8..15
                t[(j < 4) ? 4 + j : 16 + (j - 4)] = chunks[j * 64 + 32 + lane]; // K atom 1: P cols 4..7, Q cols 16..23
            }
        }
        else if(kNvf4)
        {
            // raw: [group][wire tile h = 0, 1][row 0..31][8 scales]: two words per row per wire tile, K atoms 2h and 2h + 1
#pragma unroll
            for(int j = 0; j < 12; ++j)
#pragma unroll
                for(int h = 0; h < 2; ++h)
                {
                    const bool in    = (j < 4) || (j - 4 < q_groups);
                    const uint2* grp = reinterpret_cast<const uint2*>((j < 4) ? rawp + j * 128 : rawq + (j - 4) * 128);
                    const uint2 v    = in ? grp[h * 32 + lane] : make_uint2(kNeutralSf, kNeutralSf);
                    t[(j < 4) ? (2 * h) * 4 + j : 16 + (2 * h) * 8 + (j - 4)]         = v.x;
                    t[(j < 4) ? (2 * h + 1) * 4 + j : 16 + (2 * h + 1) * 8 + (j - 4)] = v.y;
                }
        }
        else
        {
            // raw: [group][k quarter a][row 0..31][4 k-blocks]: one word per row per K atom
#pragma unroll
            for(int j = 0; j < 12; ++j)
#pragma unroll
                for(int a = 0; a < kAtomsK; ++a)
                {
                    const bool in       = (j < 4) || (j - 4 < q_groups);
                    const uint32_t* grp = (j < 4) ? rawp + j * (32 * kAtomsK) : rawq + (j - 4) * (32 * kAtomsK);
                    const int col       = (j < 4) ? a * 4 + j : 4 * kAtomsK + a * 8 + (j - 4);
                    t[col]              = in ? grp[a * 32 + lane] : kNeutralSf;
                }
        }
        const uint32_t tsf = tlane + prm.sf_tmem_base + s * prm.sf_cols;
        tmem_st_x16(tsf, t);
        if(kTWords == 24)
            tmem_st_x8(tsf + 16, t + 16);
        if(kTWords == 48)
        {
            tmem_st_x16(tsf + 16, t + 16);
            tmem_st_x16(tsf + 32, t + 32);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if(lane == 0)
        {
            if(CG == 2)
                mbar_arrive_cluster(full_leader + 8u * s);
            else
                mbar_arrive(full_leader + 8u * s);
            B200_TRACE(if(tracing && warp == 2 && g < 8) stamp(4 + 4 * g);)
        }
        return true;
    };

    if(warp == 0 || warp == 10)
    {
        // ------------------------------------------------------------------ operand producers (every CTA)
        // warp 0 loads this CTA's P tile, warp 10 its Q tile; both count their bytes on the leader's full[s]
        if(lane == 0)
        {
            const bool is_p   = (warp == 0);
            const bool is_f4  = is_p ? p_f4 : q_f4;
            const int mode    = is_p ? prm.p_mode : prm.q_mode;
            const CUtensorMap* map = is_p ? &map_p : &map_q;
            const uint32_t my_bytes = is_f4 ? 0u : (is_p ? kTileP * kTileKBytes : q_box_bytes);
            const uint32_t tile0    = smem_base + (is_p ? 0u : L.q_off);
            const uint32_t full0    = (CG == 2) ? map_to_cta(full_bar(0), 0) : full_bar(0); // the leader's barrier counts both CTAs' bytes
            const uint32_t empty0   = empty_bar(0);
            int g = 0;
            bool ok = true;
            Ring ring{0, 0};
            // One loop per operand layout, so that the per-K-tile path is a wait, an expect_tx and the tile load.
            auto run = [&](auto mode_tag) {
                constexpr int MODE = decltype(mode_tag)::value;
                B200_TRACE(if(tracing && is_p) stamp(56);)
                for(WorkIter w = first_work(); w.valid && ok; next_unit(w))
                {
                    B200_TRACE(if(tracing && is_p && w.u == cluster_id) stamp(57);)
                    const int row0 = is_p ? (w.tp * CG + static_cast<int>(crank)) * kTileP
                                          : w.tq * bn + static_cast<int>(crank) * q_rows_cta;
                    int kt         = w.it_beg;
                    for(int i = 0; i < w.n_iters; ++i, ++kt, ++g, ring.advance(S))
                    {
                        const int s = ring.s;
                        ok = bounded_wait(empty0 + 8u * s, ring.phase ^ 1u, abort_f, prm.status, ST_TIMEOUT_PRODUCER, g);
                        if(!ok)
                            break;
                        B200_TRACE(if(tracing && is_p && g == 0) stamp(58);)
                        const uint32_t dst = tile0 + s * L.stage_bytes;
                        const uint32_t bar = full0 + 8u * s;
                        if(MODE == 3)
                        {
                            // the packed e2m1 operand (always 16x16-byte tiled) lands in this CTA's staging area:
                            // 4 chunks of 16 bytes per row, counted on a local barrier for the scale warps
                            const uint32_t sbar = sfraw_bar(s);
                            mbar_arrive_expect_tx(sbar, (is_p ? kTileP : q_rows_cta) * 64u);
                            tma_load_3d(smem_base + s * L.stage_bytes + L.stg_off, map, sbar, 0, row0 >> 4, kt * 4);
                            if(CG == 1)
                                mbar_arrive_expect_tx(bar, 0u);
                            else
                                mbar_arrive_expect_tx_cluster(bar, 0u);
                        }
                        else if(CG == 1)
                        {
                            mbar_arrive_expect_tx(bar, my_bytes);
                            if(MODE == OPM_ROWMAJOR)
                                tma_load_2d(dst, map, bar, kt * kTileKBytes, row0);
                            else if(MODE == OPM_BATCHED)
                                tma_load_3d(dst, map, bar, kt * kTileKBytes, row0, w.b);
                            else if(MODE == OPM_TILE16)
                                tma_load_3d(dst, map, bar, 0, row0 >> 4, kt * (kTileKBytes / 16));
                            else
                                tma_load_4d(dst, map, bar, 0, 0, row0 >> 1, kt);
                        }
                        else
                        {
                            mbar_arrive_expect_tx_cluster(bar, my_bytes);
                            if(MODE == OPM_ROWMAJOR)
                                tma_load_2d_pair(dst, map, bar, kt * kTileKBytes, row0);
                            else if(MODE == OPM_BATCHED)
                                tma_load_3d_pair(dst, map, bar, kt * kTileKBytes, row0, w.b);
                            else if(MODE == OPM_TILE16)
                                tma_load_3d_pair(dst, map, bar, 0, row0 >> 4, kt * (kTileKBytes / 16));
                            else
                                tma_load_4d_pair(dst, map, bar, 0, 0, row0 >> 1, kt);
                        }
                        B200_TRACE(if(tracing && is_p && g < 8) stamp(2 + 4 * g);)
                    }
                }
            };
            if(is_f4)
                run(std::integral_constant<int, 3>{});
            else if(mode == OPM_ROWMAJOR)
                run(std::integral_constant<int, OPM_ROWMAJOR>{});
            else if(mode == OPM_TILE16)
                run(std::integral_constant<int, OPM_TILE16>{});
            else if(mode == OPM_BATCHED)
                run(std::integral_constant<int, OPM_BATCHED>{});
            else
                run(std::integral_constant<int, OPM_A2X128>{});
            if(*abort_f)
            {
                // give loads still in flight time to land before this CTA's shared memory is released (bounded);
                // the final CTA / cluster barrier keeps the CTAs resident meanwhile
                const uint64_t t0 = global_timer_ns();
                while(global_timer_ns() - t0 < 200000ull) {}
            }
        }
    }
    else if(warp == 11)
    {
        // ------------------------------------------------------------------ raw scale producer (every CTA)
        // (test hook: with c_wait_ctl.withhold_scales set this role issues nothing; the waits behind it then run
        // out after the shortened limit, which is how the time-out path is exercised without faulting anything)
        if(kScaled && lane == 0 && c_wait_ctl.withhold_scales == 0u)
        {
            const uint32_t sfp_bytes = 4u * kSfChunk;
            const uint32_t sfq_bytes = static_cast<uint32_t>((bn + 31) / 32) * kSfChunk;
            int g = 0;
            bool ok = true;
            Ring ring{0, 0};
            for(WorkIter w = first_work(); w.valid && ok; next_unit(w))
            {
                const int grp_p = ((w.tp * CG + static_cast<int>(crank)) * kTileP) >> 5;
                const int grp_q = (w.tq * bn) >> 5;
                int kc          = w.it_beg * kSfChunk;
                for(int i = 0; i < w.n_iters; ++i, kc += kSfChunk, ++g, ring.advance(S))
                {
                    const int s = ring.s;
                    ok = bounded_wait(empty_bar(s), ring.phase ^ 1u, abort_f, prm.status, ST_TIMEOUT_PRODUCER, 0x20000 + g);
                    if(!ok)
                        break;
                    const uint32_t stage = smem_base + s * L.stage_bytes;
                    const uint32_t bar   = sfraw_bar(s);
                    mbar_arrive_expect_tx(bar, sfp_bytes + sfq_bytes);
                    if(kNvf4) // 512-byte chunks are two 256-byte pieces of a 3-D view (a box dimension holds 256 elements)
                    {
                        tma_load_3d(stage + L.sfp_off, &map_sfp, bar, 0, kc >> 8, grp_p);
                        tma_load_3d(stage + L.sfq_off, &map_sfq, bar, 0, kc >> 8, grp_q);
                    }
                    else
                    {
                        tma_load_2d(stage + L.sfp_off, &map_sfp, bar, kc, grp_p);
                        tma_load_2d(stage + L.sfq_off, &map_sfq, bar, kc, grp_q);
                    }
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
                idesc = idesc_block_scaled(1, 1, kM, bn, !kNvf4);
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

            // The issue loop runs on one thread and must stay well under the 512 cycles the four MMAs of a stage
            // take: descriptors are a base word plus small adds, nothing is divided, nothing is re-derived.
            const uint32_t p_hi = static_cast<uint32_t>(make_smem_desc(0, p_lbo, p_sbo, p_lay) >> 32);
            const uint32_t q_hi = static_cast<uint32_t>(make_smem_desc(0, q_lbo, q_sbo, q_lay) >> 32);
            const uint32_t p_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base, p_lbo, p_sbo, p_lay));
            const uint32_t q_lo0 = static_cast<uint32_t>(make_smem_desc(smem_base + L.q_off, q_lbo, q_sbo, q_lay));
            const uint32_t stage_step = L.stage_bytes >> 4, p_step = p_adv >> 4, q_step = q_adv >> 4;
            uint32_t idk[4];
#pragma unroll
            for(int k = 0; k < 4; ++k)
                idk[k] = (KIND == KIND_BF16 || kNvf4) ? idesc
                         : (KIND == KIND_MXF4)        ? idesc_with_sf(idesc, (k & 1) * 2, (k & 1) * 2)
                                                      : idesc_with_sf(idesc, k, k);
            const uint32_t sf0 = tmem_base + prm.sf_tmem_base;
            const uint32_t full0 = full_bar(0), empty0 = empty_bar(0);

            int g = 0, uc = 0;
            bool ok = true;
            Ring ring{0, 0};
            int a = 0;
            uint32_t acc_phase = 1; // parity to wait on for "accumulator a is free"; a fresh barrier passes parity 1
            for(WorkIter w = first_work(); w.valid && ok; next_unit(w), ++uc)
            {
                const uint32_t d_col = tmem_base + a * prm.acc_stride;
                ok = bounded_wait(acc_empty_bar(a), acc_phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, 0x10000 + uc);
                if(!ok)
                    break;
                tc_fence_after_sync();
                const int n_iters = w.n_iters;
                for(int i = 0; i < n_iters; ++i, ++g, ring.advance(S))
                {
                    const int s = ring.s;
                    ok = bounded_wait(full0 + 8u * s, ring.phase, abort_f, prm.status, ST_TIMEOUT_MMA_FULL, g);
                    if(!ok)
                        break;
                    tc_fence_after_sync();
                    B200_TRACE(if(tracing && g < 8) stamp(5 + 4 * g);)
                    const uint32_t p_lo = p_lo0 + s * stage_step;
                    const uint32_t q_lo = q_lo0 + s * stage_step;
                    const uint32_t tsfp = sf0 + s * prm.sf_cols;
                    const uint32_t tsfq = tsfp + 4 * kAtomsK;
#pragma unroll
                    for(int k = 0; k < 4; ++k)
                    {
                        const uint64_t pd  = pack_u64(p_lo + k * p_step, p_hi);
                        const uint64_t qd  = pack_u64(q_lo + k * q_step, q_hi);
                        const uint32_t acc = (k > 0) ? 1u : static_cast<uint32_t>(i > 0);
                        if(CG == 1)
                        {
                            if(KIND == KIND_BF16)
                                mma_f16(d_col, pd, qd, idk[k], acc);
                            else if(KIND == KIND_MXF8 || KIND == KIND_MXF8F4)
                                mma_mxf8f6f4(d_col, pd, qd, idk[k], acc, tsfp, tsfq);
                            else if(kNvf4)
                                mma_nvf4(d_col, pd, qd, idk[k], acc, tsfp + k * 4, tsfq + k * 8);
                            else
                                mma_mxf4(d_col, pd, qd, idk[k], acc, tsfp + (k >> 1) * 4, tsfq + (k >> 1) * 8);
                        }
                        else
                        {
                            if(KIND == KIND_BF16)
                                mma_f16_2cta(d_col, pd, qd, idk[k], acc);
                            else if(KIND == KIND_MXF8 || KIND == KIND_MXF8F4)
                                mma_mxf8f6f4_2cta(d_col, pd, qd, idk[k], acc, tsfp, tsfq);
                            else if(kNvf4)
                                mma_nvf4_2cta(d_col, pd, qd, idk[k], acc, tsfp + k * 4, tsfq + k * 8);
                            else
                                mma_mxf4_2cta(d_col, pd, qd, idk[k], acc, tsfp + (k >> 1) * 4, tsfq + (k >> 1) * 8);
                        }
                    }
                    if(CG == 1)
                        tc_commit(empty0 + 8u * s);
                    else
                        tc_commit_2cta(empty0 + 8u * s, 3);
                }
                if(ok)
                {
                    if(CG == 1)
                        tc_commit(acc_full_bar(a));
                    else
                        tc_commit_2cta(acc_full_bar(a), 3);
                }
                if(++a == prm.n_acc)
                {
                    a = 0;
                    acc_phase ^= 1u;
                }
            }
            B200_TRACE(stamp(60);)
            if(!ok)
            {
                // abort: let whatever was issued finish before TMEM is released
                if(CG == 1)
                    tc_commit(drain_bar);
                else
                    tc_commit_2cta(drain_bar, 1);
                const uint64_t t0 = global_timer_ns();
                while(!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < c_wait_ctl.limit_ns) {}
            }
        }
    }
    else if(warp < 6)
    {
        // ------------------------------------------------------------------ scale warps (every CTA)
        if(kScaled)
        {
            int g = 0;
            bool ok = true;
            Ring ring{0, 0};
            for(WorkIter w = first_work(); w.valid && ok; next_iter(w), ++g, ring.advance(S))
                ok = scale_tile(ring.s, ring.phase, w.it_beg + w.i, g);
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
        const bool vec_ok = (!prm.transposed_out) && ((prm.ldo & (prm.out_mode == OUT_F32 ? 3 : 7)) == 0) && ((reinterpret_cast<uintptr_t>(prm.out) & 15) == 0) &&
                            ((prm.out_batch_stride & 7) == 0);
        // Output staging: every epilogue warp owns two 2 KB buffers (32 rows x 64 bytes) and stores them with its
        // own TMA tile stores, so the warps never wait for one another and global memory sees whole 64-byte runs.
        const bool use_tma   = prm.tma_store != 0;
        const uint32_t epi_warp_bytes = prm.epi_bufs == 2 ? 8192u : 4096u;
        uint8_t* epi_gen     = smem_gen + L.epi_off + (warp - 6) * epi_warp_bytes;
        const uint32_t epi_s = smem_base + L.epi_off + (warp - 6) * epi_warp_bytes;
        int ebuf             = 0;
        uint32_t wbuf        = 0; // wide stores: which of the two 4 KB buffers comes next (0 when there is only one)
        if(use_tma && lane == 0)
            tma_prefetch_desc(&map_out);
        uint32_t epi_phase = 0;
        int uc = 0;
        bool ok = true;
        Ring wring{0, 0};
        int wseq = 0; // stages seen by the widening loop
        const uint32_t full_lead = (CG == 2) ? map_to_cta(full_bar(0), 0) : full_bar(0);
        for(WorkIter w = first_work(); w.valid && ok; next_unit(w), ++uc)
        {
            if(kMixed)
            {
                // Mixed kind: these four warps first widen the packed e2m1 operand of every K tile of this unit to
                // e4m3 in the MMA's un-swizzled layout (staging [4 chunks][rows][16 B], 32 codes each -> tile
                // [8 chunks][rows][16 B]) while the scale warps feed the scales, then turn to the unit's epilogue.
                const int rows = p_f4 ? kTileP : q_rows_cta;
                const int tid  = (warp - 6) * 32 + lane;
                // 128-row tiles: warps 6,7 take the even stages of the ring sequence and warps 8,9 the odd ones (six items
                // per thread), so that the fixed cost of a stage (barrier wait, fence, arrival) is paid per two tiles
                const bool by_pairs = (rows == kTileP);
                const int my_pair   = (warp - 6) >> 1;
                const int tid2      = ((warp - 6) & 1) * 32 + lane;
                for(int i = 0; i < w.n_iters && ok; ++i, wring.advance(S), ++wseq)
                {
                    if(by_pairs && (wseq & 1) != my_pair)
                        continue;
                    const int s = wring.s;
                    ok = bounded_wait(sfraw_bar(s), wring.phase, abort_f, prm.status, ST_TIMEOUT_SFWARP, 0x10000 + i);
                    ok = __all_sync(0xffffffffu, ok);
                    if(!ok)
                        break;
                    B200_TRACE(if(tracing && warp == 6 && lane == 0 && uc == 0 && i < 8) stamp(34 + 2 * i);)
                    uint8_t* stage   = smem_gen + s * L.stage_bytes;
                    const uint4* src = reinterpret_cast<const uint4*>(stage + L.stg_off);
                    uint4* dst       = reinterpret_cast<uint4*>(stage + (p_f4 ? 0u : L.q_off));
                    if(by_pairs)
                    {
                        // 128 rows: items (16-byte k chunk u, row); chunks 0..2 here (rows tid2 and tid2 + 64), chunk 3 by the
                        // scale warps, whose own work per stage is shorter.  All loads first, so that their latencies
                        // overlap instead of adding up
                        uint4 v[6];
#pragma unroll
                        for(int u = 0; u < 6; ++u)
                            v[u] = src[(u >> 1) * kTileP + (u & 1) * 64 + tid2];
#pragma unroll
                        for(int u = 0; u < 6; ++u)
                        {
                            uint4 o0, o1;
                            e2m1x8_to_e4m3x8(v[u].x, o0.x, o0.y);
                            e2m1x8_to_e4m3x8(v[u].y, o0.z, o0.w);
                            e2m1x8_to_e4m3x8(v[u].z, o1.x, o1.y);
                            e2m1x8_to_e4m3x8(v[u].w, o1.z, o1.w);
                            dst[(2 * (u >> 1)) * kTileP + (u & 1) * 64 + tid2]     = o0;
                            dst[(2 * (u >> 1) + 1) * kTileP + (u & 1) * 64 + tid2] = o1;
                        }
                    }
                    else
                        for(int it = tid; it < rows * 4; it += 128)
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
                    __syncwarp();
                    if(lane == 0)
                    {
                        if(CG == 2)
                            mbar_arrive_cluster(full_lead + 8u * s);
                        else
                            mbar_arrive(full_lead + 8u * s);
                        B200_TRACE(if(tracing && warp == 6 && uc == 0 && i < 8) stamp(35 + 2 * i);)
                    }
                }
                if(!ok)
                    break;
            }
            const int a       = uc % prm.n_acc;
            const int p       = (w.tp * CG + static_cast<int>(crank)) * kTileP + p_local;
            const int row_q0  = w.tq * bn;
            const int slot    = ((w.b * prm.tiles_p + w.tp) * prm.tiles_q + w.tq) * CG + static_cast<int>(crank); // ticket / partial slot of this CTA tile
            // this pair's output and bias (batched problems)
            const bool out_f16 = (prm.out_mode == OUT_F16);
            void* const out_b  = static_cast<uint8_t*>(prm.out) +
                                static_cast<size_t>(w.b) * static_cast<size_t>(prm.out_batch_stride) * (prm.out_mode == OUT_F32 ? 4u : 2u);
            const void* const bias_b = prm.bias == nullptr ? nullptr
                                       : static_cast<const uint8_t*>(prm.bias) + static_cast<size_t>(w.b) * static_cast<size_t>(prm.bias_batch_stride) * (prm.bias_is_bf16 ? 2u : 4u);
            ok = bounded_wait(acc_full_bar(a), (uc / prm.n_acc) & 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, uc);
            ok = __all_sync(0xffffffffu, ok);
            if(!ok)
                break;
            tc_fence_after_sync();
            B200_TRACE(if(warp == 6 && lane == 0 && uc == 0) stamp(61);)
            const uint32_t tacc = tlane + a * prm.acc_stride;
            bool is_last        = !split;
            auto release_acc = [&]() {
                tc_fence_before_sync();
                __syncwarp();
                if(lane == 0)
                {
                    if(CG == 2)
                        mbar_arrive_cluster(acc_empty_remote + 8u * a);
                    else
                        mbar_arrive(acc_empty_bar(a));
                }
            };

            // Cluster-split tile.  Up to 4 slices: reduce-scatter, CTA z adds up and stores rows [z * per, (z + 1) * per)
            // of the tile (per = 128 / csplit: whole epilogue warps) and receives the other slices' partial sums of
            // them; 8 slices: the first CTA reduces the whole tile.  A warp whose rows belong to another CTA sends its
            // partial accumulator to that CTA's shared memory ([source slice][row][bn floats]); the bytes are counted on
            // that CTA's red barrier and nothing is waited for.
            const bool scatter    = csplit > 1 && csplit <= 4;
            const uint32_t per    = scatter ? static_cast<uint32_t>(kTileP / csplit) : static_cast<uint32_t>(kTileP);
            const uint32_t owner  = scatter ? static_cast<uint32_t>(p_local) / per : 0u;
            const uint32_t prow   = static_cast<uint32_t>(p_local) - owner * per;
            if(csplit > 1)
                cluster_wait_acquire(); // every CTA of the cluster has initialised its barriers (long ago: they all ran a main loop since)
            if(csplit > 1 && warp == 6 && lane == 0 && (scatter || zrank == 0))
                mbar_arrive_expect_tx(red_bar, static_cast<uint32_t>(csplit - 1) * per * static_cast<uint32_t>(bn) * 4u);
            if(csplit > 1 && zrank != owner)
            {
                const uint32_t src    = zrank < owner ? zrank : zrank - 1u; // this slice's place among the owner's sources
                const uint32_t dst_row = map_to_cta(smem_base + L.red_off, owner) + (src * per + prow) * static_cast<uint32_t>(bn) * 4u;
                const uint32_t dst_bar = map_to_cta(red_bar, owner);
                for(int c = 0; c < n_chunks; ++c)
                {
                    uint32_t r[32];
                    if(chunk == 32)
                        tmem_ld_x32(tacc + c * 32, r);
                    else
                        tmem_ld_x16(tacc + c * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for(int j = 0; j < 32; j += 4)
                        if(j < chunk)
                            st_async_v4(dst_row + static_cast<uint32_t>(c * chunk + j) * 4u, r[j], r[j + 1], r[j + 2], r[j + 3], dst_bar);
                }
                release_acc();
                continue;
            }

            if(split)
            {
                float* mine = prm.ws_partial + (static_cast<size_t>(slot) * splits + w.z) * (static_cast<size_t>(bn) * kTileP);
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
                release_acc(); // the accumulator is drained: hand it back before the reduction
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
                // finish one chunk of columns: alpha / bias, bf16, store
                auto finish = [&](float (&v)[32], const int c) {
                    const int q_first = row_q0 + c * chunk;
                    if(bias_b != nullptr)
                    {
                        const float bp = (!prm.bias_on_q && p < prm.rows_p) ? load_bias(bias_b, prm.bias_is_bf16, p) : 0.f;
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                        {
                            float b = bp;
                            if(prm.bias_on_q)
                                b = (j < chunk && q_first + j < prm.rows_q) ? load_bias(bias_b, prm.bias_is_bf16, q_first + j) : 0.f;
                            v[j] = prm.alpha * v[j] + prm.beta * b;
                        }
                    }
                    else if(prm.alpha != 1.0f)
                    {
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                            v[j] *= prm.alpha;
                    }
                    if(use_tma)
                    {
                        if(lane == 0)
                            bulk_wait_group_read<1>(); // the store issued from this buffer two chunks ago has read it
                        __syncwarp();
                        uint8_t* buf = epi_gen + ebuf * 2048;
                        if(!prm.transposed_out)
                        {
                            // row = lane, 64 bytes (32 columns); 16-byte pieces swizzled (64B mode) against bank conflicts
#pragma unroll
                            for(int j = 0; j < 4; ++j)
                                *reinterpret_cast<uint4*>(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) * 16)) =
                                    make_uint4(pack_out16x2(v[8 * j], v[8 * j + 1], out_f16), pack_out16x2(v[8 * j + 2], v[8 * j + 3], out_f16),
                                               pack_out16x2(v[8 * j + 4], v[8 * j + 5], out_f16), pack_out16x2(v[8 * j + 6], v[8 * j + 7], out_f16));
                        }
                        else
                        {
                            // row = output row q (chunk of them), 64 bytes = this warp's 32 values of p
#pragma unroll
                            for(int j = 0; j < 32; ++j)
                                if(j < chunk)
                                    reinterpret_cast<uint16_t*>(buf)[j * 32 + lane] = cvt_out16(v[j], out_f16);
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        const int p_warp0 = (w.tp * CG + static_cast<int>(crank)) * kTileP + quarter * 32;
                        if(lane == 0 && p_warp0 < prm.rows_p && q_first < prm.rows_q) // partly outside: the store clips
                        {
                            if(!prm.transposed_out)
                                tma_store_2d(&map_out, epi_s + ebuf * 2048, q_first * 2, p_warp0);
                            else
                                tma_store_2d(&map_out, epi_s + ebuf * 2048, p_warp0 * 2, q_first);
                            bulk_commit_group();
                        }
                        ebuf ^= 1;
                    }
                    else if(p < prm.rows_p)
                    {
                        if(!prm.transposed_out)
                        {
                            const size_t at = static_cast<size_t>(p) * prm.ldo + q_first;
                            if(prm.out_mode == OUT_F32)
                            {
                                float* dst = static_cast<float*>(out_b) + at;
                                if(vec_ok && q_first + chunk <= prm.rows_q)
                                {
#pragma unroll
                                    for(int j = 0; j < 32; j += 4)
                                        if(j < chunk)
                                            *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                }
                                else
                                {
#pragma unroll
                                    for(int j = 0; j < 32; ++j)
                                        if(j < chunk && q_first + j < prm.rows_q)
                                            dst[j] = v[j];
                                }
                            }
                            else
                            {
                                uint16_t* dst = static_cast<uint16_t*>(out_b) + at;
                                if(vec_ok && q_first + chunk <= prm.rows_q)
                                {
#pragma unroll
                                    for(int j = 0; j < 32; j += 8)
                                        if(j < chunk)
                                            *reinterpret_cast<uint4*>(dst + j) =
                                                make_uint4(pack_out16x2(v[j], v[j + 1], out_f16), pack_out16x2(v[j + 2], v[j + 3], out_f16),
                                                           pack_out16x2(v[j + 4], v[j + 5], out_f16), pack_out16x2(v[j + 6], v[j + 7], out_f16));
                                }
                                else
                                {
#pragma unroll
                                    for(int j = 0; j < 32; ++j)
                                        if(j < chunk && q_first + j < prm.rows_q)
                                            dst[j] = cvt_out16(v[j], out_f16);
                                }
                            }
                        }
                        else
                        {
#pragma unroll
                            for(int j = 0; j < 32; ++j)
                            {
                                const int q = q_first + j;
                                if(j < chunk && q < prm.rows_q)
                                    store_out(out_b, static_cast<size_t>(q) * prm.ldo + p, v[j], prm.out_mode);
                            }
                        }
                    }
                };
                if(prm.out_mode >= OUT_E2M1)
                {
                    // Re-quantising epilogue (row-major output, no K split, tile width a multiple of 128): the thread's row
                    // goes out 128 columns at a time.  e4m3 + UE8M0: the block's maximum first (one pass over the TMEM
                    // columns), scale byte = RoundUp(amax / 448) with amax clamped below by FLT_MIN, then a second pass
                    // converts (TMEM can be read twice; 128 fp32 values would not fit the registers).  Packed e2m1: a
                    // saturating round-to-nearest-even cast, no scale.  Same arithmetic as the activation quantiser.
                    uint8_t* const out8 = static_cast<uint8_t*>(prm.out);
                    const bool row_ok   = p < prm.rows_p;
                    const float al      = prm.alpha; // the product of the per-tensor scales of NVFP4 inputs; 1 otherwise
                    for(int b128 = 0; b128 < (bn >> 7); ++b128)
                    {
                        const int q_first = row_q0 + b128 * 128;
                        const bool col_ok = q_first < prm.rows_q;
                        float rscale      = 1.f;
                        if(prm.out_mode == OUT_MXFP8)
                        {
                            float amax   = 0.f;
                            bool has_nan = false;
#pragma unroll 1
                            for(int c = 0; c < 4; ++c)
                            {
                                uint32_t r[32];
                                tmem_ld_x32(tacc + b128 * 128 + c * 32, r);
                                tmem_ld_wait();
#pragma unroll
                                for(int j = 0; j < 32; ++j)
                                {
                                    const float x = __uint_as_float(r[j]) * al;
                                    amax          = fmaxf(amax, fabsf(x));
                                    has_nan |= (x != x);
                                }
                            }
                            amax = has_nan ? __uint_as_float(0x7FC00000u) : fmaxf(amax, 1.17549435e-38f);
                            const uint32_t qb   = __float_as_uint(__fdiv_rn(amax, 448.0f));
                            const uint32_t ex   = (qb >> 23) & 0xFFu;
                            const uint32_t byte = ex + (((qb & 0x7FFFFFu) != 0u && ex < 0xFFu) ? 1u : 0u);
                            rscale = __uint_as_float(byte == 0xFFu ? 0x7F800001u : (byte == 254u ? 0x00400000u : ((254u - byte) << 23)));
                            if(row_ok && col_ok)
                            {
                                const int m = p, j = q_first >> 7;
                                prm.out_scale[((static_cast<size_t>(m >> 6) * prm.out_scale_cols + j) * 16 + (m & 15)) * 4 + ((m & 63) >> 4)] = static_cast<uint8_t>(byte);
                            }
                        }
#pragma unroll 1
                        for(int c = 0; c < 4; ++c)
                        {
                            uint32_t r[32];
                            tmem_ld_x32(tacc + b128 * 128 + c * 32, r);
                            tmem_ld_wait();
                            if(al != 1.0f)
                            {
#pragma unroll
                                for(int j = 0; j < 32; ++j)
                                    r[j] = __float_as_uint(__uint_as_float(r[j]) * al);
                            }
                            if(prm.out_mode == OUT_MXFP8)
                            {
                                uint32_t wds[8];
#pragma unroll
                                for(int h = 0; h < 8; ++h)
                                {
                                    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
                                        make_float2(__uint_as_float(r[4 * h]) * rscale, __uint_as_float(r[4 * h + 1]) * rscale), __NV_SATFINITE, __NV_E4M3);
                                    const __nv_fp8x2_storage_t hi2 = __nv_cvt_float2_to_fp8x2(
                                        make_float2(__uint_as_float(r[4 * h + 2]) * rscale, __uint_as_float(r[4 * h + 3]) * rscale), __NV_SATFINITE, __NV_E4M3);
                                    wds[h] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi2) << 16);
                                }
                                if(row_ok && q_first + c * 32 < prm.rows_q)
                                {
                                    uint4* dst = reinterpret_cast<uint4*>(out8 + static_cast<size_t>(p) * prm.ldo + q_first + c * 32);
                                    dst[0]     = make_uint4(wds[0], wds[1], wds[2], wds[3]);
                                    dst[1]     = make_uint4(wds[4], wds[5], wds[6], wds[7]);
                                }
                            }
                            else
                            {
                                uint32_t wds[4];
#pragma unroll
                                for(int h = 0; h < 4; ++h)
                                {
                                    uint32_t packed = 0;
#pragma unroll
                                    for(int i = 0; i < 4; ++i)
                                        packed |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(
                                                      make_float2(__uint_as_float(r[8 * h + 2 * i]), __uint_as_float(r[8 * h + 2 * i + 1])), __NV_E2M1, cudaRoundNearest))
                                                  << (8 * i);
                                    wds[h] = packed;
                                }
                                if(row_ok && q_first + c * 32 < prm.rows_q)
                                    *reinterpret_cast<uint4*>(out8 + static_cast<size_t>(p) * prm.ldo + ((q_first + c * 32) >> 1)) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
                            }
                        }
                    }
                    release_acc();
                }
                else if(!split && prm.tma_store == 2)
                {
                    // Wide path (row-major output, tile width a multiple of 64): 64 columns per step, so that the
                    // one warp per scheduler that runs this code has long runs of independent instructions: one
                    // TMEM load, 32 conversions, 8 shared-memory stores (128B-swizzled rows), one tile store.
                    const bool epi_math = (bias_b != nullptr) || (prm.alpha != 1.0f);
                    const int p_warp0   = (w.tp * CG + static_cast<int>(crank)) * kTileP + quarter * 32;
                    const int n64       = bn >> 6;
                    for(int c = 0; c < n64; ++c)
                    {
                        uint32_t r[64];
                        tmem_ld_x64(tacc + c * 64, r);
                        tmem_ld_wait();
                        if(c == n64 - 1)
                            release_acc(); // every column of this accumulator is in registers now
                        const int q_first = row_q0 + c * 64;
                        if(epi_math)
                        {
                            // three plain loops (a per-element test of the bias form inside one loop cost 17 % of a
                            // 16384 x 7168 x 7168 NVFP4 GEMM, whose per-tensor factors arrive as alpha)
                            const float al = prm.alpha;
                            if(bias_b == nullptr)
                            {
#pragma unroll
                                for(int j = 0; j < 64; ++j)
                                    r[j] = __float_as_uint(al * __uint_as_float(r[j]));
                            }
                            else if(!prm.bias_on_q)
                            {
                                const float bb = prm.beta * ((p < prm.rows_p) ? load_bias(bias_b, prm.bias_is_bf16, p) : 0.f);
#pragma unroll
                                for(int j = 0; j < 64; ++j)
                                    r[j] = __float_as_uint(al * __uint_as_float(r[j]) + bb);
                            }
                            else
                            {
#pragma unroll
                                for(int j = 0; j < 64; ++j)
                                {
                                    const float b = (q_first + j < prm.rows_q) ? load_bias(bias_b, prm.bias_is_bf16, q_first + j) : 0.f;
                                    r[j] = __float_as_uint(al * __uint_as_float(r[j]) + prm.beta * b);
                                }
                            }
                        }
                        // the store that last used this buffer has read it (the previous store with one buffer, the one
                        // before it with two: then a store's read latency no longer sits between two TMEM loads)
                        if(lane == 0)
                        {
                            if(prm.epi_bufs == 2)
                                bulk_wait_group_read<1>();
                            else
                                bulk_wait_group_read<0>();
                        }
                        __syncwarp();
                        uint8_t* row = epi_gen + wbuf + lane * 128;
                        if(out_f16)
                        {
#pragma unroll
                            for(int j = 0; j < 8; ++j)
                                *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) * 16)) =
                                    make_uint4(pack_f16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                                               pack_f16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                                               pack_f16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                                               pack_f16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
                        }
                        else
                        {
#pragma unroll
                            for(int j = 0; j < 8; ++j)
                                *reinterpret_cast<uint4*>(row + ((j ^ (lane & 7)) * 16)) =
                                    make_uint4(pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                                               pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                                               pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                                               pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if(lane == 0 && p_warp0 < prm.rows_p && q_first < prm.rows_q)
                        {
                            tma_store_2d(&map_out, epi_s + wbuf, q_first * 2, p_warp0);
                            bulk_commit_group();
                        }
                        if(prm.epi_bufs == 2)
                            wbuf ^= 4096u;
                    }
                }
                else if(!split)
                {
                    for(int c = 0; c < n_chunks; ++c)
                    {
                        uint32_t r[32];
                        if(chunk == 32)
                            tmem_ld_x32(tacc + c * 32, r);
                        else
                            tmem_ld_x16(tacc + c * 16, r);
                        tmem_ld_wait();
                        if(c == n_chunks - 1)
                            release_acc(); // every column of this accumulator is in registers now
                        float v[32];
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                            v[j] = __uint_as_float(r[j]);
                        if(csplit > 1)
                        {
                            if(c == 0)
                            {
                                ok = bounded_wait(red_bar, uc & 1, abort_f, prm.status, ST_TIMEOUT_EPILOGUE, 0x3000 + uc);
                                ok = __all_sync(0xffffffffu, ok);
                                if(!ok)
                                    break;
                            }
                            const float4* red = reinterpret_cast<const float4*>(smem_gen + L.red_off);
                            for(int z = 0; z < csplit - 1; ++z)
                            {
                                const float4* row = red + (static_cast<size_t>(z * per + prow) * bn + c * chunk) / 4;
#pragma unroll
                                for(int j = 0; j < 32; j += 4)
                                    if(j < chunk)
                                    {
                                        const float4 t = row[j / 4];
                                        v[j] += t.x;
                                        v[j + 1] += t.y;
                                        v[j + 2] += t.z;
                                        v[j + 3] += t.w;
                                    }
                            }
                        }
                        finish(v, c);
                    }
                }
                else
                {
                    for(int c = 0; c < n_chunks; ++c)
                    {
                        float v[32];
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
                        finish(v, c);
                    }
                }
                B200_TRACE(if(warp == 6 && lane == 0 && uc == 0) stamp(59);)
                if(split && warp == 6 && lane == 0)
                    prm.ws_counter[slot] = 0; // ready for the next launch
            }
        }
        // the tile stores have read their shared-memory source before the CTA retires and its shared memory is handed
        // on; their global writes need not be waited for (they are part of the grid's memory operations, which complete
        // before anything ordered after the grid runs), and waiting would add the store's full latency to the kernel's tail
        if(use_tma && lane == 0)
            bulk_wait_group_read<0>();
        B200_TRACE(if(warp == 6 && lane == 0) stamp(62);)
        B200_TRACE(if(lane == 0) stamp(43 + (warp - 6));)
        tc_fence_before_sync();
    }

    B200_TRACE(if(lane == 0 && warp < 6) stamp(47 + warp);)
    B200_TRACE(if(lane == 0 && warp >= 10) stamp(43 + warp);)
    __syncthreads();
    B200_TRACE(if(threadIdx.x == 0) stamp(55);)
    // A CTA pair stays together to the end: the partner's MMAs and commits touch this CTA's shared memory and
    // barriers.  The CTAs of a cluster K split need no such rendezvous: the only remote traffic into a CTA are the
    // partial sums it owns, and its epilogue has waited for every byte of them (red barrier) before it got here.
    if(CG == 2)
        cluster_sync_all();
    B200_TRACE(if(threadIdx.x == 0) stamp(63);)
    B200_TRACE(if(prm.trace != nullptr && threadIdx.x == 0 && blockIdx.x < 160) prm.trace[65 + 2 * blockIdx.x] = global_timer_ns();)
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
