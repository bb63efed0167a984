// Host side of the tcgen05 GEMM: tensor-map construction, configuration choice, per-stream
// split-K workspace, launch.  No torch types; only the CUDA runtime (the one driver entry point
// needed, cuTensorMapEncodeTiled, is resolved at run time so the library loads without libcuda).
#include "launch.h"
#include "gemm_persistent.cuh"
#include "gemm_decode.cuh"
#include "gemm_blockscale.cuh"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

namespace b200 {

// ---------------------------------------------------------------------------------------------
// driver entry point
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if(e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr)
            fail("cuTensorMapEncodeTiled is not available from the CUDA driver (", cudaGetErrorString(e), ")");
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

static CUtensorMap encode_map(const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                              const cuuint32_t* box, CUtensorMapSwizzle swz, const char* what)
{
    CUtensorMap m;
    cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
    CUresult r = encode_tiled_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, static_cast<cuuint32_t>(rank),
                                   const_cast<void*>(base), dims, strides_bytes, box, elem_strides,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if(r != CUDA_SUCCESS)
    {
        std::ostringstream os;
        os << "tensor map for " << what << " rejected (CUresult " << static_cast<int>(r) << "): base=" << base << " dims=";
        for(int i = 0; i < rank; ++i)
            os << dims[i] << (i + 1 < rank ? "x" : "");
        os << " strides=";
        for(int i = 0; i + 1 < rank; ++i)
            os << strides_bytes[i] << (i + 2 < rank ? "," : "");
        os << " box=";
        for(int i = 0; i < rank; ++i)
            os << box[i] << (i + 1 < rank ? "x" : "");
        fail(os.str());
    }
    return m;
}

// Operand tile map; box_rows rows by box_kbytes (128, or 64 for a packed e2m1 operand of the mixed kind)
// bytes of K per load.
static CUtensorMap operand_map(const Operand& op, int box_rows, const char* what, int box_kbytes = kTileKBytes)
{
    B200_CHECK(box_kbytes == kTileKBytes || op.mode == OPM_TILE16, what, ": a packed e2m1 operand must be 16x16-byte tiled");
    B200_CHECK((reinterpret_cast<uintptr_t>(op.ptr) & 15) == 0, what, ": base address must be 16-byte aligned");
    if(op.mode == OPM_ROWMAJOR)
    {
        B200_CHECK(op.ld_bytes % 16 == 0, what, ": row pitch must be a multiple of 16 bytes (got ", op.ld_bytes, ")");
        cuuint64_t dims[2]    = {static_cast<cuuint64_t>(op.kbytes), static_cast<cuuint64_t>(op.rows)};
        cuuint64_t strides[1] = {static_cast<cuuint64_t>(op.ld_bytes)};
        cuuint32_t box[2]     = {kTileKBytes, static_cast<cuuint32_t>(box_rows)};
        return encode_map(op.ptr, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, what);
    }
    if(op.mode == OPM_BATCHED)
    {
        // [batch][rows][K bytes]: the row-major tile of matrix b is box (128 B, rows, 1) at coordinate (k, row, b); rows past
        // the end of one matrix are zero-filled, never taken from the next one
        B200_CHECK(op.ld_bytes % 16 == 0 && op.batch_stride_bytes % 16 == 0, what, ": row pitch and batch stride must be multiples of 16 bytes");
        B200_CHECK(op.batch_stride_bytes > 0, what, ": internal: batch stride missing");
        cuuint64_t dims[3]    = {static_cast<cuuint64_t>(op.kbytes), static_cast<cuuint64_t>(op.rows), static_cast<cuuint64_t>(op.batch)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(op.ld_bytes), static_cast<cuuint64_t>(op.batch_stride_bytes)};
        cuuint32_t box[3]     = {kTileKBytes, static_cast<cuuint32_t>(box_rows), 1};
        return encode_map(op.ptr, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, what);
    }
    if(op.mode == OPM_TILE16)
    {
        B200_CHECK(op.rows % 16 == 0 && op.kbytes % 32 == 0, what,
                   ": a (16,16)-shuffled operand needs rows % 16 == 0 and K bytes % 32 == 0 (got ", op.rows, " x ",
                   op.kbytes, ")");
        B200_CHECK(box_rows % 16 == 0, what, ": internal: box rows must be a multiple of 16");
        // [rows/16][kbytes/16][256 B]; smem wants [k chunk][row][16 B], so the row-block index runs
        // faster than the k-chunk index in the box.
        cuuint64_t dims[3]    = {256, static_cast<cuuint64_t>(op.rows / 16), static_cast<cuuint64_t>(op.kbytes / 16)};
        cuuint64_t strides[2] = {static_cast<cuuint64_t>(op.kbytes) * 16, 256};
        cuuint32_t box[3]     = {256, static_cast<cuuint32_t>(box_rows / 16), static_cast<cuuint32_t>(box_kbytes / 16)};
        return encode_map(op.ptr, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, what);
    }
    B200_CHECK(op.mode == OPM_A2X128, what, ": unknown operand mode ", op.mode);
    B200_CHECK(op.rows % 2 == 0 && op.kbytes % 128 == 0, what,
               ": the (m/2,k/128,2,128) tiling needs rows % 2 == 0 and K bytes % 128 == 0");
    B200_CHECK(box_rows % 2 == 0, what, ": internal: box rows must be even");
    cuuint64_t dims[4]    = {128, 2, static_cast<cuuint64_t>(op.rows / 2), static_cast<cuuint64_t>(op.kbytes / 128)};
    cuuint64_t strides[3] = {128, static_cast<cuuint64_t>(op.kbytes) * 2, 256};
    cuuint32_t box[4]     = {128, 2, static_cast<cuuint32_t>(box_rows / 2), 1};
    return encode_map(op.ptr, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, what);
}

// Scale map: one row per 32-row group, `chunk` wire bytes per group per K tile.
static CUtensorMap scale_map(const ScaleOperand& sf, int chunk, int groups_per_tile, const char* what)
{
    B200_CHECK((reinterpret_cast<uintptr_t>(sf.ptr) & 15) == 0, what, ": base address must be 16-byte aligned");
    B200_CHECK(sf.padded_rows % 32 == 0, what, ": scale rows must be padded to a multiple of 32 (got ", sf.padded_rows, ")");
    const cuuint64_t row_bytes = static_cast<cuuint64_t>(sf.padded_cols) * 32;
    if(chunk > 256)
    {
        // a box dimension holds at most 256 elements: a 512-byte chunk (NVFP4) is two 256-byte pieces of a 3-D view
        // [group][row bytes / 256][256], which lands in shared memory in the same order as the 2-D form would
        B200_CHECK(chunk == 512 && row_bytes % 256 == 0, what, ": internal: scale chunk ", chunk);
        cuuint64_t dims3[3]    = {256, row_bytes / 256, static_cast<cuuint64_t>(sf.padded_rows / 32)};
        cuuint64_t strides3[2] = {256, row_bytes};
        cuuint32_t box3[3]     = {256, 2, static_cast<cuuint32_t>(groups_per_tile)};
        return encode_map(sf.ptr, 3, dims3, strides3, box3, CU_TENSOR_MAP_SWIZZLE_NONE, what);
    }
    cuuint64_t dims[2]    = {row_bytes, static_cast<cuuint64_t>(sf.padded_rows / 32)};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2]     = {static_cast<cuuint32_t>(chunk), static_cast<cuuint32_t>(groups_per_tile)};
    return encode_map(sf.ptr, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, what);
}

// ---------------------------------------------------------------------------------------------
// per-device / per-stream state
// ---------------------------------------------------------------------------------------------
struct StreamWorkspace
{
    float* partial        = nullptr;
    size_t partial_bytes  = 0;
    unsigned int* counter = nullptr;
    void* widened         = nullptr; // e4m3 copy of a packed e2m1 weight (mixed kind, tall problems)
    size_t widened_bytes  = 0;
    void* relaid          = nullptr; // block scales re-laid from e8m0_shuffle to the (m/32,k/4,32,4) order (MXFP4, tall problems)
    size_t relaid_bytes   = 0;
};
constexpr int kCounterSlots = 1 << 16;

struct DeviceState
{
    int sm_count         = 0;
    int smem_optin       = 0;
    unsigned int* status = nullptr;
    unsigned int* status_host = nullptr; // pinned host word the kernels copy the first failure code to; read before every launch
    WaitControl wait_ctl{kWaitLimitNs, nullptr, 0u};
    unsigned long long* trace = nullptr; // AITER_B200_TRACING builds only
    std::map<cudaStream_t, StreamWorkspace> ws;
    // Buffers that were outgrown.  A CUDA graph captured earlier may still hold their addresses, so they are never
    // freed while the process lives: replaying such a graph keeps writing into memory this library still owns.
    std::vector<void*> retired;
};

static std::mutex g_mutex;
static std::map<int, DeviceState> g_devices;
static std::atomic<unsigned long long> g_launches{0};

static DeviceState& device_state(int device)
{
    // caller holds g_mutex and has made `device` current
    auto it = g_devices.find(device);
    if(it != g_devices.end())
        return it->second;
    DeviceState st;
    cudaDeviceProp prop;
    B200_CUDA(cudaGetDeviceProperties(&prop, device));
    B200_CHECK(prop.major == 10, "this library only runs on sm_100 class GPUs (device ", device, " is sm_", prop.major,
               prop.minor, ")");
    st.sm_count   = prop.multiProcessorCount;
    st.smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
    B200_CUDA(cudaMalloc(&st.status, 4 * sizeof(unsigned int)));
    B200_CUDA(cudaMemset(st.status, 0, 4 * sizeof(unsigned int)));
    // one pinned host word, mapped into the device: a kernel whose wait runs out stores its code there too, so
    // the next call on this device can refuse to launch without a device round trip
    void* host_word = nullptr;
    if(cudaHostAlloc(&host_word, sizeof(unsigned int), cudaHostAllocMapped) == cudaSuccess)
    {
        st.status_host  = static_cast<unsigned int*>(host_word);
        *st.status_host = 0u;
        void* dev_view  = nullptr;
        if(cudaHostGetDevicePointer(&dev_view, host_word, 0) == cudaSuccess)
            st.wait_ctl.host_mirror = static_cast<unsigned int*>(dev_view);
    }
    else
        cudaGetLastError();
    B200_CUDA(cudaMemcpyToSymbol(c_wait_ctl, &st.wait_ctl, sizeof(WaitControl)));
    return g_devices.emplace(device, st).first->second;
}

// A wait that ran out in an earlier kernel left its code in the pinned host word: refuse further launches until the
// caller has fetched (and thereby cleared) the record.  Caller holds g_mutex.
static void require_healthy(const DeviceState& st, int device)
{
    if(st.status_host != nullptr)
    {
        const unsigned int code = *reinterpret_cast<volatile unsigned int*>(st.status_host);
        B200_CHECK(code == 0u, "an earlier kernel on device ", device, " gave up on a wait (status code 0x", std::hex, code, std::dec,
                   "); its output is incomplete. Read and clear the record with aiter_b200_device_status before launching again");
    }
}

// Retire an outgrown buffer instead of freeing it (see DeviceState::retired).
static void retire(DeviceState& st, void* p)
{
    if(p != nullptr)
        st.retired.push_back(p);
}

static StreamWorkspace& stream_workspace(DeviceState& st, cudaStream_t stream, size_t partial_bytes)
{
    StreamWorkspace& w = st.ws[stream];
    const bool need_counter = (w.counter == nullptr);
    const bool need_grow    = (partial_bytes > w.partial_bytes);
    if(need_counter || need_grow)
    {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(stream, &cap);
        B200_CHECK(cap == cudaStreamCaptureStatusNone,
                   "split-K workspace must grow (", partial_bytes, " bytes) but the stream is being captured; run this "
                   "shape once outside capture first");
    }
    if(need_counter)
    {
        B200_CUDA(cudaMalloc(&w.counter, kCounterSlots * sizeof(unsigned int)));
        B200_CUDA(cudaMemset(w.counter, 0, kCounterSlots * sizeof(unsigned int)));
    }
    if(need_grow)
    {
        // grow geometrically, so that a sequence of ever larger shapes retires only a few buffers
        size_t bytes = std::max(std::max(partial_bytes, static_cast<size_t>(8) << 20), 2 * w.partial_bytes);
        retire(st, w.partial);
        w.partial       = nullptr;
        w.partial_bytes = 0;
        B200_CUDA(cudaMalloc(&w.partial, bytes));
        w.partial_bytes = bytes;
    }
    return w;
}

int device_sm_count(int device)
{
    int prev = 0;
    B200_CUDA(cudaGetDevice(&prev));
    B200_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lk(g_mutex);
    int n = device_state(device).sm_count;
    cudaSetDevice(prev);
    return n;
}

void read_device_status(int device, unsigned int out_words[4])
{
    int prev = 0;
    B200_CUDA(cudaGetDevice(&prev));
    B200_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lk(g_mutex);
    DeviceState& st = device_state(device);
    B200_CUDA(cudaDeviceSynchronize());
    B200_CUDA(cudaMemcpy(out_words, st.status, 4 * sizeof(unsigned int), cudaMemcpyDeviceToHost));
    B200_CUDA(cudaMemset(st.status, 0, 4 * sizeof(unsigned int)));
    if(st.status_host != nullptr)
        *st.status_host = 0u;
    if(out_words[0] != 0u)
    {
        // a kernel that gave up may have left split-K tickets half counted: later launches must start from zero
        for(auto& kv : st.ws)
            if(kv.second.counter != nullptr)
                B200_CUDA(cudaMemset(kv.second.counter, 0, kCounterSlots * sizeof(unsigned int)));
    }
    cudaSetDevice(prev);
}

void set_wait_control(int device, unsigned long long limit_ns, int withhold_scales)
{
    B200_CHECK(limit_ns >= 1000ull * 1000ull && limit_ns <= 10ull * kWaitLimitNs, "wait limit must be between 1 ms and 10 s");
    int prev = 0;
    B200_CUDA(cudaGetDevice(&prev));
    B200_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lk(g_mutex);
    DeviceState& st = device_state(device);
    B200_CUDA(cudaDeviceSynchronize()); // no kernel may be reading the constants while they change
    st.wait_ctl.limit_ns        = limit_ns;
    st.wait_ctl.withhold_scales = withhold_scales ? 1u : 0u;
    B200_CUDA(cudaMemcpyToSymbol(c_wait_ctl, &st.wait_ctl, sizeof(WaitControl)));
    cudaSetDevice(prev);
}

unsigned long long launch_count() { return g_launches.load(); }
void count_launch() { g_launches.fetch_add(1); }

// ---------------------------------------------------------------------------------------------
// configuration menu / heuristic
// ---------------------------------------------------------------------------------------------
static const int kBnMenu[] = {16, 32, 64, 128, 256, 192, 224, 96, 160};

static int kernel_kind_of(int problem_kind)
{
    switch(problem_kind)
    {
    case PK_BF16: return KIND_BF16;
    case PK_MXFP8: return KIND_MXF8;
    case PK_MXFP4: return KIND_MXF4;
    case PK_MXF8F4: return KIND_MXF8F4;
    case PK_NVFP4: return KIND_NVF4;
    default: fail("problem kind ", problem_kind, " has no kernel in this build");
    }
}

static int max_stages(int bn, int cg, int smem_limit, int f4_operand, int scaled, int epi_stage, int csplit = 1)
{
    for(int s = kMaxStages; s >= 1; --s)
        if(static_cast<int>(make_persistent_smem(bn, cg, s, f4_operand, scaled, epi_stage, csplit).total) + 1024 <= smem_limit)
            return s;
    return 0;
}

// Tall MXFP4 problems with e8m0_shuffle scales: that byte order costs the scale warps a transpose through shared
// memory on every K tile; re-laying both scale tensors once into the (m/32,k/4,32,4) order (a few MB) lets the
// main loop run the cheaper path.
constexpr long long kScalePrepassMinM = 1024;
constexpr long long kScalePrepassMinK = 4096; // the two extra launches (~6 us) must be won back over the K loop ...
                                              // ... which on a tall problem (tall_problem) they are at any K >= 1024

// A tall MXFP4 / NVFP4 problem: enough output tiles that the per-call re-layout of e8m0_shuffle scales (two small
// launches) and the narrower two-accumulator tile pay back even at a short K.  Measured with the tuner at K = 1536 / 2048:
// 16384 x 7168 142 -> 133 us, 4096 x 24576 98.5 -> 92.3 us; 2048 x 24576 a tie; 4096 x 7168 42.9 -> 44.1 us (not tall).
static bool tall_problem(long long M, long long N) { return M >= 8192 || (M >= 4096 && M * N >= 8192LL * 7168); }

void choose_config(int kind, long long M, long long N, long long K, int num_sms, KernelConfig& cfg)
{
    if(cfg.swap < 0)
    {
        cfg.swap = (M <= 64) ? 1 : 0;
        // 65..256 rows of the scaled kinds (not the mixed one, whose decode form is bound by its widening): the decode
        // kernel on tiles of 64 rows, each on the same weight tile, while all those CTAs are resident at once (two per SM);
        // measured against the persistent kernel's 128-wide tiles: MXFP4 256 x 7168 x 2048 10.5 -> 8.2 us, 256 x 8192 x 8192
        // 23.9 -> 20.8 us, MXFP8 128 x 4096 x 4096 15.7 -> 12.4 us; 256 x 24576 x 1536 (768 CTAs) 15.6 -> 20.3 us
        // Tiles of 128 rows instead (the tuner's choices over the reference's model shapes): for up to 128 rows of a large
        // weight (N >= 5120, N x K >= 48 M elements) one tile with four stages, a CTA alone on its SM (128 x 7168 x 16384
        // 24.8 -> 22.9 us); for 129..256 rows where four tiles of 64 per weight tile no longer fit the machine but two of 128 do.
        if(M > 64 && M <= 256 && cfg.bn <= 0 && cfg.cg <= 0 && (kind == PK_MXFP8 || kind == PK_MXFP4 || kind == PK_NVFP4))
        {
            const long long tiles_p = (N + kTileP - 1) / kTileP;
            if(M <= 128 && N >= 5120 && N * K >= 48LL * 1024 * 1024 && tiles_p <= num_sms && cfg.stages <= 0)
            {
                cfg.swap          = 1;
                cfg.bn            = 128;
                cfg.decode_stages = 4;
            }
            else if(tiles_p * ((M + 63) / 64) <= 2LL * num_sms)
            {
                cfg.swap = 1;
                cfg.bn   = 64;
            }
            else if(tiles_p * ((M + 127) / 128) <= 2LL * num_sms)
            {
                cfg.swap = 1;
                cfg.bn   = 128;
            }
        }
    }
    const long long rows_q = cfg.swap ? M : N;
    const long long rows_p = cfg.swap ? N : M;
    const bool bn_was_open = (cfg.bn <= 0);
    if(cfg.bn <= 0)
    {
        if(cfg.swap)
            cfg.bn = rows_q <= 16 ? 16 : rows_q <= 32 ? 32 : rows_q <= 64 ? 64 : rows_q <= 128 ? 128 : 256;
        else
        {
            // largest tile whose grid still covers half the machine
            // (the tuner's tables agree: a 256-wide tile on half the SMs beats a 128-wide one on all of them)
            cfg.bn = 256;
            const long long tiles_p = (rows_p + kTileP - 1) / kTileP;
            while(cfg.bn > 64 && tiles_p * ((rows_q + cfg.bn - 1) / cfg.bn) < num_sms / 2)
                cfg.bn >>= 1;
            if(rows_q < cfg.bn)
                cfg.bn = rows_q <= 16 ? 16 : rows_q <= 32 ? 32 : rows_q <= 64 ? 64 : rows_q <= 128 ? 128 : 256;
        }
    }
    const bool four_bit = (kind == PK_MXFP4 || kind == PK_NVFP4);
    if(bn_was_open && cfg.cg <= 0 && !cfg.swap && rows_p >= 512 && rows_q >= 192)
    {
        // CTA pairs (each SM stages half of the Q tile per flop) pay from about two dozen 256 x 256 tiles on: the tuner's
        // tables name a pair tile for every such shape of the reference's model list, down to 512 x 2560
        const long long pair_rows = (rows_p + 2 * kTileP - 1) / (2 * kTileP);
        if(pair_rows * ((rows_q + 255) / 256) >= 24)
        {
            cfg.cg = 2;
            cfg.bn = 256;
            if(four_bit)
            {
                // 256 x 256 (TMEM for one accumulator: the epilogue is exposed) against 256 x 192 (two accumulators, 7/8
                // of the operand bytes for 3/4 of the flops): waves over the SM pairs x time per tile, fitted to the
                // tuner's measurements in units of 10 ns.  Where the scales are in the cheap order (tall problems:
                // re-laid once per call; NVFP4's wire order) a tile takes 0.42 / 0.40 us per K tile of 256 elements plus
                // 2.0 / 0.6 us; otherwise the scale warps set the pace and both widths take 0.38 us per K tile plus
                // 3.1 us, so only the number of waves (then the padding of the last tile) decides.
                const long long k_tiles = (K + 255) / 256;
                const bool cheap_scales = (kind == PK_NVFP4) || (rows_p >= kScalePrepassMinM && K % 256 == 0 && K >= (tall_problem(rows_p, rows_q) ? 1024 : kScalePrepassMinK));
                const long long t256    = cheap_scales ? k_tiles * 42 + 200 : k_tiles * 38 + 310;
                const long long t192    = cheap_scales ? k_tiles * 40 + 57 : k_tiles * 38 + 310;
                const long long pairs   = std::max(num_sms / 2, 1);
                auto waves = [&](long long bn) { return (pair_rows * ((rows_q + bn - 1) / bn) + pairs - 1) / pairs; };
                auto pad   = [&](long long bn) { return (rows_q + bn - 1) / bn * bn - rows_q; };
                const long long c256 = waves(256) * t256, c192 = waves(192) * t192;
                if(c192 < c256 || (c192 == c256 && pad(192) <= pad(256)))
                    cfg.bn = 192;
            }
        }
    }
    if(cfg.cg <= 0)
    {
        // (below that: pairs only where the chosen tile still gives every SM pair work)
        const long long pair_tiles = ((rows_p + 2 * kTileP - 1) / (2 * kTileP)) * ((rows_q + cfg.bn - 1) / cfg.bn);
        cfg.cg = (!cfg.swap && cfg.bn >= 128 && cfg.bn % 32 == 0 && rows_p >= 512 && pair_tiles * 2 >= num_sms) ? 2 : 1;
    }
    const int elems_per_iter = (kind == PK_BF16) ? 64 : ((kind == PK_MXFP4 || kind == PK_NVFP4) ? 256 : 128);
    const long long k_iters  = (K + elems_per_iter - 1) / elems_per_iter;
    if(cfg.log2_splitk < 0)
    {
        const long long tiles = ((rows_p + kTileP * cfg.cg - 1) / (kTileP * cfg.cg)) * ((rows_q + cfg.bn - 1) / cfg.bn) * cfg.cg;
        int l2 = 0;
        // split while the grid under-fills the machine and every split keeps >= 4 K iterations.  Decode tiles (the small
        // kernel: two CTAs per SM, K split over a cluster of at most four) may fill the machine twice.
        const bool decode  = cfg.swap && cfg.cg == 1 && cfg.bn <= 64;
        const long long cap = decode ? 2LL * num_sms : num_sms;
        const int max_l2    = decode ? 2 : 5;
        // Fitted to the tuner's choices over the reference's model shapes: pair tiles never split (no shape where the
        // workspace split paid); single-CTA tiles of a problem with 512 rows or more only for slices of 24 K tiles; decode
        // tiles of 64 rows stream 24 KB per K tile and want slices of 6 K tiles while the split grid still fits one CTA
        // per SM, 16 beyond.  Clusters do not pack the machine to the last slot (they may not straddle a GPC): a split
        // into clusters of four may take 7/8 of the two-CTAs-per-SM capacity (64 x 9216 x 16384: 288 CTAs in clusters of four
        // 34 us, in pairs 23.8 us).
        auto min_iters = [&](int next_l2) -> long long {
            if(decode && cfg.bn == 64)
                return tiles * (1LL << next_l2) <= num_sms ? 6 : 16;
            if(!cfg.swap && rows_p >= 512)
                return 24;
            return 4;
        };
        auto capacity = [&](int next_l2) -> long long { return decode && next_l2 >= 2 ? cap - cap / 8 : cap; };
        while(cfg.cg == 1 && l2 < max_l2 && tiles * (2LL << l2) <= capacity(l2 + 1) && (k_iters >> (l2 + 1)) >= min_iters(l2 + 1))
            ++l2;
        cfg.log2_splitk = l2;
    }
    if(cfg.stages <= 0)
    {
        int s        = max_stages(cfg.bn, cfg.cg, 227 * 1024, kind == PK_MXF8F4 ? (cfg.swap ? 1 : 2) : 0, sf_unit_of(kernel_kind_of(kind)), true);
        cfg.stages   = s > kMaxStages ? kMaxStages : s;
    }
}

std::string config_name(const KernelConfig& cfg)
{
    char buf[64];
    std::snprintf(buf, sizeof(buf), "tc5_%dx%d_%c_s%d", 128 * (cfg.cg > 0 ? cfg.cg : 1), cfg.bn, cfg.swap ? 't' : 'n', cfg.stages);
    return buf;
}

bool parse_config_name(const char* name, KernelConfig& cfg)
{
    if(name == nullptr || name[0] == 0)
        return false;
    int bm = 0, bn = 0, stages = 0, l2 = -1, consumed = 0;
    char sw = 0;
    if(std::sscanf(name, "tc5_%dx%d_%c_s%d%n", &bm, &bn, &sw, &stages, &consumed) != 4 || (bm != 128 && bm != 256))
        return false;
    if(name[consumed] != 0) // optional "_k<log2 of the K split>"
    {
        int more = 0;
        if(std::sscanf(name + consumed, "_k%d%n", &l2, &more) != 1 || name[consumed + more] != 0 || l2 < 0 || l2 > 8)
            return false;
    }
    bool ok = false;
    for(int b : kBnMenu)
        ok |= (b == bn);
    if(!ok || (sw != 'n' && sw != 't') || stages < 0 || stages > kMaxStages)
        return false;
    cfg.bn     = bn;
    cfg.swap   = (sw == 't');
    cfg.stages = stages; // 0 = as many as fit
    cfg.cg     = bm / 128;
    if(l2 >= 0)
        cfg.log2_splitk = l2;
    return true;
}

// kernelId = pair * 1000 + swap * 100 + index(bn) * 10 + stages   (stages 0 = as many as fit)
bool config_from_id(int kernel_id, KernelConfig& cfg)
{
    if(kernel_id < 0)
        return false;
    const int pair = kernel_id / 1000, swap = (kernel_id / 100) % 10, bi = (kernel_id / 10) % 10, st = kernel_id % 10;
    if(pair > 1 || swap > 1 || bi >= static_cast<int>(sizeof(kBnMenu) / sizeof(int)) || st > kMaxStages)
        return false;
    cfg.cg     = pair + 1;
    cfg.swap   = swap;
    cfg.bn     = kBnMenu[bi];
    cfg.stages = st;
    return true;
}

const char* kernel_menu_text()
{
    static std::string text = [] {
        std::ostringstream os;
        os << "kernelName = tc5_<128|256>x<bn>_<n|t>_s<stages>[_k<log2 K split>]; kernelId = pair*1000 + swap*100 + bn_index*10 + stages (0 = max)\n"
           << "  256-row tiles (pair = 1) run on CTA pairs (cta_group::2)\n";
        for(int swap = 0; swap < 2; ++swap)
            for(size_t bi = 0; bi < sizeof(kBnMenu) / sizeof(int); ++bi)
                os << "  id " << swap * 100 + bi * 10 << "..: tile 128x" << kBnMenu[bi]
                   << (swap ? "  weights on the 128-row slot (decode shapes), transposed store"
                            : "  activations on the 128-row slot")
                   << "\n";
        return os.str();
    }();
    return text.c_str();
}

// ---------------------------------------------------------------------------------------------
// launch
// ---------------------------------------------------------------------------------------------
static bool pdl_disabled()
{
    static const bool off = (std::getenv("AITER_B200_NO_PDL") != nullptr);
    return off;
}

// Raise the dynamic shared-memory limit once per device for one kernel; `attr_done` is the caller's
// per-instantiation flag array (caller holds g_mutex).
template <typename Kernel>
static void raise_smem_limit(Kernel kernel, bool (&attr_done)[64])
{
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    if(dev < 0 || dev >= 64 || !attr_done[dev])
    {
        B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        if(dev >= 0 && dev < 64)
            attr_done[dev] = true;
    }
}

template <int KIND, int SFW, int CG>
static void launch_persistent(int ctas, size_t smem, cudaStream_t stream, const CUtensorMap& mp, const CUtensorMap& mq,
                              const CUtensorMap& msp, const CUtensorMap& msq, const CUtensorMap& mo, const PersistentParams& prm)
{
    auto kernel = gemm_persistent_kernel<KIND, SFW, CG>;
    static bool attr_done[64] = {};
    raise_smem_limit(kernel, attr_done);
    cudaLaunchConfig_t lc{};
    lc.gridDim          = dim3(ctas, 1, 1);
    lc.blockDim         = dim3(kPersistentThreads, 1, 1);
    lc.dynamicSmemBytes = smem;
    lc.stream           = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG * (prm.csplit > 1 ? prm.csplit : 1);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // this kernel's prologue may start while the previous kernel of the stream drains (it waits with
    // griddepcontrol.wait before its first global access)
    attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs    = attr;
    lc.numAttrs = pdl_disabled() ? 1 : 2;
    B200_CUDA(cudaLaunchKernelEx(&lc, kernel, mp, mq, msp, msq, mo, prm));
    g_launches.fetch_add(1);
}

template <int KIND, int SFW>
static void launch_persistent_cg(int cg, int ctas, size_t smem, cudaStream_t stream, const CUtensorMap& mp,
                                 const CUtensorMap& mq, const CUtensorMap& msp, const CUtensorMap& msq,
                                 const CUtensorMap& mo, const PersistentParams& prm)
{
    if(cg == 2)
        launch_persistent<KIND, SFW, 2>(ctas, smem, stream, mp, mq, msp, msq, mo, prm);
    else
        launch_persistent<KIND, SFW, 1>(ctas, smem, stream, mp, mq, msp, msq, mo, prm);
}

static bool cluster_split_disabled()
{
    static const bool off = (std::getenv("AITER_B200_NO_CLUSTER_SPLIT") != nullptr);
    return off;
}

#ifdef AITER_B200_TRACING
constexpr int kTraceCtas  = 160;
constexpr int kTraceWords = 64 + 2 * kTraceCtas;

static void print_trace(DeviceState& st, const GemmProblem& prob, const KernelConfig& cfg, int tiles_p, int tiles_q, int splits,
                        int stages)
{
    // debugging aid: timestamp record of the first CTA, SM clock cycles relative to kernel entry
    static unsigned long long t[kTraceWords];
    B200_CUDA(cudaStreamSynchronize(prob.stream));
    B200_CUDA(cudaMemcpy(t, st.trace, sizeof(t), cudaMemcpyDeviceToHost));
    std::fprintf(stderr, "[trace] kind %d %lldx%lldx%lld %s tiles %dx%d splits %d stages %d:", prob.kind, prob.M, prob.N, prob.K,
                 config_name(cfg).c_str(), tiles_p, tiles_q, splits, stages);
    for(int i = 0; i < 64; ++i)
        if(t[i] != 0)
            std::fprintf(stderr, " %d:%lld", i, static_cast<long long>(t[i] - t[0]));
    // every CTA's begin / end on the global nanosecond timer, relative to the earliest begin
    unsigned long long first = ~0ull;
    for(int b = 0; b < kTraceCtas; ++b)
        if(t[64 + 2 * b] != 0 && t[64 + 2 * b] < first)
            first = t[64 + 2 * b];
    std::fprintf(stderr, "\n[trace] cta begin-end ns:");
    for(int b = 0; b < kTraceCtas; ++b)
        if(t[64 + 2 * b] != 0)
            std::fprintf(stderr, " %d:%lld-%lld", b, static_cast<long long>(t[64 + 2 * b] - first),
                         static_cast<long long>(t[65 + 2 * b] - first));
    std::fprintf(stderr, "\n");
}
#endif // AITER_B200_TRACING

// Packed e2m1 weight in the 16x16-byte tiled layout -> e4m3 in the same tiling (twice the K chunks).  Exact: every
// e2m1 value is an e4m3 value.  One thread per 16-byte chunk (32 codes of one row).
__global__ void widen_e2m1_tile16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long row_blocks, int chunks_in)
{
    const long long total = row_blocks * chunks_in * 16;
    for(long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
        i += static_cast<long long>(gridDim.x) * blockDim.x)
    {
        const int r         = static_cast<int>(i & 15);
        const long long t   = i >> 4;
        const int kc        = static_cast<int>(t % chunks_in);
        const long long nb  = t / chunks_in;
        const uint4 v       = src[i];
        uint4 o0, o1;
        e2m1x8_to_e4m3x8(v.x, o0.x, o0.y);
        e2m1x8_to_e4m3x8(v.y, o0.z, o0.w);
        e2m1x8_to_e4m3x8(v.z, o1.x, o1.y);
        e2m1x8_to_e4m3x8(v.w, o1.z, o1.w);
        const long long base = (nb * (2LL * chunks_in) + 2LL * kc) * 16 + r;
        dst[base]      = o0;
        dst[base + 16] = o1;
    }
}

// e8m0_shuffle scale bytes -> (m/32, k/4, 32, 4) order, one thread per output word (one row, four K blocks).
// src byte index: (m/32 * cols_pad) * 32 + (k/8) * 256 + (k%4) * 64 + (m%16) * 4 + ((k%8)/4) * 2 + (m%32)/16.
__global__ void relay_e8m0_shuffle_kernel(const uint8_t* __restrict__ src, uint32_t* __restrict__ dst, int groups, int cols_pad, int kblocks)
{
    const int atoms       = kblocks / 4;
    const long long total = static_cast<long long>(groups) * atoms * 32;
    for(long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
        i += static_cast<long long>(gridDim.x) * blockDim.x)
    {
        const int r        = static_cast<int>(i & 31);
        const long long t  = i >> 5;
        const int a        = static_cast<int>(t % atoms);
        const long long g  = t / atoms;
        const uint8_t* p   = src + (g * cols_pad) * 32 + (a >> 1) * 256 + (r & 15) * 4 + (a & 1) * 2 + (r >> 4);
        dst[i]             = static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[64]) << 8) | (static_cast<uint32_t>(p[128]) << 16) |
                             (static_cast<uint32_t>(p[192]) << 24);
    }
}

static bool panel_order_disabled()
{
    static const bool off = (std::getenv("AITER_B200_NO_PANELS") != nullptr);
    return off;
}

static bool relay_prepass_disabled()
{
    static const bool off = (std::getenv("AITER_B200_NO_SCALE_PREPASS") != nullptr);
    return off;
}

static bool widen_prepass_disabled()
{
    static const bool off = (std::getenv("AITER_B200_NO_WIDEN_PREPASS") != nullptr);
    return off;
}

static void launch_gemm_locked(const GemmProblem& prob);

// ---------------------------------------------------------------------------------------------
// decode shapes: the small kernel of gemm_decode.cuh
// ---------------------------------------------------------------------------------------------
static bool decode_kernel_disabled()
{
    static const bool off = (std::getenv("AITER_B200_NO_DECODE_KERNEL") != nullptr);
    return off;
}

static bool decode_mixed_disabled()
{
    static const bool off = (std::getenv("AITER_B200_DECODE_NO_MIXED") != nullptr);
    return off;
}

constexpr uint32_t kDecodeBarrierBytes = 256; // the decode kernel's barriers and flags (gemm_decode.cuh)

struct DecodeLayout
{
    uint32_t stage_bytes, q_off, sfp_off, sfq_off, cook_off, stg_off, red_off, bar_off, total;
};

// scaled: raw scale bytes per 32-row group per K tile in units of 256 (decode_sf_unit)
static DecodeLayout make_decode_layout(int bn, int stages, int csplit, int scaled, bool cook, bool mixed)
{
    DecodeLayout L;
    const uint32_t q_groups = static_cast<uint32_t>((bn + 31) / 32);
    L.q_off       = kTileP * kTileKBytes;
    L.sfp_off     = L.q_off + static_cast<uint32_t>(bn) * kTileKBytes;
    L.sfq_off     = L.sfp_off + 1024u * static_cast<uint32_t>(scaled);
    L.cook_off    = L.sfq_off + 256u * q_groups * static_cast<uint32_t>(scaled); // (the activation scales' box holds q_groups groups)
    L.stg_off     = L.cook_off + (cook ? 2048u : 0u);      // re-ordered scales: 2 sides x up to 2 K atoms x 512 bytes
    const uint32_t used = L.stg_off + (mixed ? kTileP * 64u : 0u); // mixed kind: the packed e2m1 weight tile, 128 rows x 64 bytes
    L.stage_bytes = (used + 1023u) & ~1023u;               // every stage starts on the swizzle atom's 1024-byte boundary
    L.red_off     = L.stage_bytes * static_cast<uint32_t>(stages);
    L.bar_off     = L.red_off + (csplit > 1 ? static_cast<uint32_t>(csplit - 1) * static_cast<uint32_t>(kTileP / csplit) * static_cast<uint32_t>(bn) * 4u : 0u);
    L.total       = L.bar_off + kDecodeBarrierBytes;
    // The barrier block fits into the last stage's padding where that has room to spare; with 64 activation rows and
    // e8m0_shuffle scales this is what lets a fourth stage in beside a second CTA on the SM
    // (never inside the first 32 KB of the ring, which the epilogue reuses as its staging buffers)
    if(csplit == 1 && L.stage_bytes - used >= kDecodeBarrierBytes && L.red_off - kDecodeBarrierBytes >= 32768u)
    {
        L.bar_off = L.red_off - kDecodeBarrierBytes;
        L.total   = L.red_off;
    }
    return L;
}

template <int KIND, int SFW>
static void launch_decode_instance(int ctas, int tiles_q, int csplit, size_t smem, cudaStream_t stream, const CUtensorMap& mp, const CUtensorMap& mq,
                                   const CUtensorMap& msp, const CUtensorMap& msq, const CUtensorMap& mo, const DecodeParams& prm)
{
    auto kernel = gemm_decode_kernel<KIND, SFW>;
    static bool attr_done[64] = {};
    {
        int dev = 0;
        B200_CUDA(cudaGetDevice(&dev));
        if(dev >= 0 && dev < 64 && !attr_done[dev]) // two CTAs of up to 113 KB each per SM need the largest shared-memory carve-out
            B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    }
    raise_smem_limit(kernel, attr_done);
    cudaLaunchConfig_t lc{};
    lc.gridDim          = dim3(ctas, tiles_q, 1);
    lc.blockDim         = dim3(kDecodeThreads, 1, 1);
    lc.dynamicSmemBytes = smem;
    lc.stream           = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs    = attr;
    lc.numAttrs = pdl_disabled() ? 1 : 2;
    B200_CUDA(cudaLaunchKernelEx(&lc, kernel, mp, mq, msp, msq, mo, prm));
    g_launches.fetch_add(1);
}

// Launches the decode kernel if the problem and configuration fit it; returns false otherwise (the persistent kernel
// then serves the call).  Caller holds g_mutex and has made the device current.
static bool try_launch_decode(const GemmProblem& prob, const KernelConfig& cfg, int kkind, DeviceState& st)
{
    // what the caller's configuration asked for, else what the heuristic did (0: this kernel's own choice)
    const int named_stages = prob.cfg.stages > 0 ? prob.cfg.stages : cfg.decode_stages;
    // one tile of activation rows, or up to four tiles of 64 / two of 128 (each a CTA of its own on the same weight tile);
    // a 128-column tile named with more than four stages stays with the persistent kernel
    const int tiles_q = static_cast<int>((prob.M + cfg.bn - 1) / std::max(cfg.bn, 1));
    if(decode_kernel_disabled() || !cfg.swap || cfg.cg != 1 || cfg.bn > 128 || cfg.bn % 16 != 0 || (cfg.bn > 64 && cfg.bn != 128) ||
       (tiles_q > 1 && (cfg.bn < 64 || tiles_q * cfg.bn > 256)) || (cfg.bn == 128 && named_stages > 4) || prob.scratch != nullptr ||
       prob.out_mode != OUT_BF16 || prob.batch > 1 || prob.noscale)
        return false;
    const bool mixed = (kkind == KIND_MXF8F4);
    if(mixed && decode_mixed_disabled())
        return false;
    const int num_k_iters = static_cast<int>((prob.act.kbytes + kTileKBytes - 1) / kTileKBytes);
    int csplit            = 1 << cfg.log2_splitk;
    while(csplit > num_k_iters)
        csplit >>= 1;
    if(csplit > 4)
        return false; // wider K splits stay with the persistent kernel (workspace or 8-CTA cluster)
    const bool scaled = (kkind != KIND_BF16);
    const int bn      = cfg.bn;
    // e8m0_shuffle scales: the four scale warps share the byte transpose and the MMA thread copies the result to TMEM
    // (tcgen05.cp); the (m/32,k/4,32,4) order needs no transpose, there the warps write TMEM themselves
    static const bool no_cp = (std::getenv("AITER_B200_DECODE_NO_CP") != nullptr);
    const bool cook = scaled && !no_cp && prob.wgt_sf.wire == SFW_E8M0_SHUFFLE;
    // as many stages as keep two CTAs on an SM (228 KB, of which each CTA also takes 1 KB of system space), unless the
    // configuration names a count
    int stages = 0;
    const int smem_cap = named_stages > 0 ? st.smem_optin : (228 * 1024) / 2 - 1024;
    for(int s2 = std::min(named_stages > 0 ? named_stages : kDecodeMaxStages, kDecodeMaxStages); s2 >= 2; --s2)
        if(static_cast<int>(make_decode_layout(bn, s2, csplit, decode_sf_unit(kkind), cook, mixed).total) + 1024 <= smem_cap)
        {
            stages = s2;
            break;
        }
    if(stages == 0)
        return false;
    stages                  = std::min(stages, std::max(2, (num_k_iters + csplit - 1) / csplit));
    const DecodeLayout L    = make_decode_layout(bn, stages, csplit, decode_sf_unit(kkind), cook, mixed);
    const Operand& P        = prob.wgt;
    const Operand& Q        = prob.act;
    if(mixed)
        B200_CHECK(Q.kbytes == 2 * P.kbytes && P.mode == OPM_TILE16,
                   "mixed MXFP8 x MXFP4: the weight must be packed e2m1 in the 16x16-byte tiled layout");
    else
        B200_CHECK(P.kbytes == Q.kbytes, "operands disagree on K bytes: ", P.kbytes, " vs ", Q.kbytes);
    CUtensorMap mp  = operand_map(P, kTileP, "weight operand", mixed ? 64 : kTileKBytes);
    CUtensorMap mq  = operand_map(Q, bn, "activation operand");
    CUtensorMap msp = mp, msq = mq;
    int sfw = SFW_NONE;
    const int kblocks = static_cast<int>(prob.K / 32);
    if(scaled)
    {
        const ScaleOperand& SP = prob.wgt_sf;
        const ScaleOperand& SQ = prob.act_sf;
        const int atoms_k      = (kkind == KIND_NVF4) ? 4 : ((kkind == KIND_MXF4) ? 2 : 1);
        B200_CHECK(SP.wire == SQ.wire && SP.wire != SFW_NONE, "both scale tensors must use the same wire layout");
        sfw = SP.wire;
        B200_CHECK(sfw != SFW_E8M0_SHUFFLE || kkind == KIND_MXF4, "the e8m0_shuffle scale layout is only wired for MXFP4");
        B200_CHECK(kkind != KIND_NVF4 || sfw == SFW_G1250, "NVFP4 scales arrive in tiles of 32 rows x 8 scales");
        const int chunk = (sfw == SFW_E8M0_SHUFFLE) ? 256 : 128 * atoms_k;
        msp = scale_map(SP, chunk, 4, "weight scales");
        msq = scale_map(SQ, chunk, (bn + 31) / 32, "activation scales");
        const long long need_cols = (kkind == KIND_NVF4) ? prob.K / 16 : (sfw == SFW_E8M0_SHUFFLE) ? (kblocks + 7) / 8 * 8 : kblocks;
        B200_CHECK(SP.padded_cols >= need_cols && SQ.padded_cols >= need_cols, "scale tensors have too few columns: need ",
                   need_cols, ", got ", SP.padded_cols, " and ", SQ.padded_cols);
        B200_CHECK(SP.padded_rows >= (P.rows + 31) / 32 * 32 && SQ.padded_rows >= (Q.rows + 31) / 32 * 32, "scale tensors have too few rows");
        if(sfw == SFW_G1250)
            B200_CHECK(prob.K % (kkind == KIND_MXF8 || kkind == KIND_MXF8F4 ? 128 : 256) == 0, "K must be a multiple of ",
                       (kkind == KIND_MXF8 || kkind == KIND_MXF8F4 ? 128 : 256), " for this scale layout");
    }
    DecodeParams prm{};
    prm.rows_p      = static_cast<int>(P.rows);
    prm.rows_q      = static_cast<int>(Q.rows);
    prm.num_k_iters = num_k_iters;
    prm.kblocks     = kblocks;
    prm.bn          = bn;
    prm.stages      = stages;
    prm.p_mode      = P.mode; // (mixed kind: the widened tile has the same 16x16-byte tiled arrangement)
    prm.q_mode      = Q.mode;
    prm.csplit      = csplit;
    prm.stage_bytes = L.stage_bytes;
    prm.q_off       = L.q_off;
    prm.sfp_off     = L.sfp_off;
    prm.sfq_off     = L.sfq_off;
    prm.cook_off    = L.cook_off;
    prm.stg_off     = L.stg_off;
    prm.sf_via_cp   = cook ? 1 : 0;
    prm.red_off     = L.red_off;
    prm.bar_off     = L.bar_off;
    prm.out         = static_cast<__nv_bfloat16*>(prob.out);
    prm.ldo         = prob.ldo;
    prm.bias        = prob.bias;
    prm.bias_is_bf16 = prob.bias_is_bf16;
    prm.alpha       = prob.alpha;
    prm.beta        = prob.beta;
    prm.status      = st.status;
#ifdef AITER_B200_TRACING
    static const bool trace_on = (std::getenv("AITER_B200_TRACE") != nullptr);
    static const int trace_every = std::getenv("AITER_B200_TRACE_EVERY") ? std::atoi(std::getenv("AITER_B200_TRACE_EVERY")) : 1;
    static int trace_seq = 0;
    bool trace_print = false;
    if(trace_on)
    {
        if(st.trace == nullptr)
        {
            B200_CUDA(cudaMalloc(&st.trace, kTraceWords * sizeof(unsigned long long)));
            B200_CUDA(cudaMemset(st.trace, 0, kTraceWords * sizeof(unsigned long long)));
        }
        prm.trace   = st.trace;
        trace_print = (++trace_seq % std::max(trace_every, 1) == 0);
    }
#endif
    int cols = 32;
    while(cols < bn + stages * decode_sf_cols(kkind))
        cols <<= 1;
    prm.tmem_cols = cols;
    CUtensorMap mo = mp;
    prm.tma_store  = ((reinterpret_cast<uintptr_t>(prob.out) & 15) == 0) && (prob.ldo % 8 == 0) ? 1 : 0;
    if(prm.tma_store)
    {
        // bf16 [M][N] seen as bytes; a warp's box is its 32 output columns by the tile's bn rows
        const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(prob.N) * 2, static_cast<cuuint64_t>(prob.M)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(prob.ldo) * 2};
        const cuuint32_t box[2]     = {64u, static_cast<cuuint32_t>(std::min(bn, 64))}; // (a 128-column tile leaves in two chunks)
        mo = encode_map(prob.out, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, "output");
    }
    const int tiles_p = static_cast<int>((P.rows + kTileP - 1) / kTileP);
    const int ctas    = tiles_p * csplit;
    const size_t smem = L.total + 1024;
    if(kkind == KIND_BF16)
        launch_decode_instance<KIND_BF16, SFW_NONE>(ctas, tiles_q, csplit, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_MXF8 && sfw == SFW_G1250)
        launch_decode_instance<KIND_MXF8, SFW_G1250>(ctas, tiles_q, csplit, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_MXF4 && sfw == SFW_E8M0_SHUFFLE)
        launch_decode_instance<KIND_MXF4, SFW_E8M0_SHUFFLE>(ctas, tiles_q, csplit, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_MXF4 && sfw == SFW_G1250)
        launch_decode_instance<KIND_MXF4, SFW_G1250>(ctas, tiles_q, csplit, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_MXF8F4 && sfw == SFW_G1250)
        launch_decode_instance<KIND_MXF8F4, SFW_G1250>(ctas, tiles_q, csplit, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_NVF4 && sfw == SFW_G1250)
        launch_decode_instance<KIND_NVF4, SFW_G1250>(ctas, tiles_q, csplit, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else
        fail("no decode kernel instance for kind ", kkind, " with scale layout ", sfw);
#ifdef AITER_B200_TRACING
    if(trace_print)
        print_trace(st, prob, cfg, tiles_p, tiles_q, csplit, stages);
#endif
    return true;
}

// Tall mixed MXFP8 x MXFP4 problems: widening the weight once (N x K bytes through HBM) is cheaper than widening
// every tile of it in shared memory M / 256 times; the GEMM itself then runs as plain MXFP8.  Below the
// threshold, inside stream capture without a buffer, or with caller-provided scratch the in-kernel path runs.
constexpr long long kWidenPrepassMinM = 512;

void launch_gemm(const GemmProblem& prob)
{
    if(prob.M == 0 && prob.N > 0 && prob.K > 0)
        return; // no activation rows: nothing to compute, the (empty) output is already complete
    if(prob.kind == PK_MXFP4 && prob.M >= kScalePrepassMinM && prob.scratch == nullptr && prob.act_sf.wire == SFW_E8M0_SHUFFLE &&
       prob.wgt_sf.wire == SFW_E8M0_SHUFFLE && prob.K % 256 == 0 && prob.K >= (tall_problem(prob.M, prob.N) ? 1024 : kScalePrepassMinK) &&
       !relay_prepass_disabled())
    {
        int prev_dev = 0;
        B200_CUDA(cudaGetDevice(&prev_dev));
        if(prev_dev != prob.device)
            B200_CUDA(cudaSetDevice(prob.device));
        struct Restore
        {
            int prev, cur;
            ~Restore()
            {
                if(prev != cur)
                    cudaSetDevice(prev);
            }
        } restore{prev_dev, prob.device};
        const int kblocks    = static_cast<int>(prob.K / 32);
        const long long ga   = (prob.M + 31) / 32, gw = (prob.N + 31) / 32;
        const bool fits      = prob.act_sf.padded_rows >= ga * 32 && prob.wgt_sf.padded_rows >= gw * 32 &&
                               prob.act_sf.padded_cols >= kblocks && prob.wgt_sf.padded_cols >= kblocks &&
                               prob.act_sf.padded_cols % 8 == 0 && prob.wgt_sf.padded_cols % 8 == 0;
        uint32_t* relaid = nullptr;
        if(fits)
        {
            std::lock_guard<std::mutex> lk(g_mutex);
            DeviceState& st    = device_state(prob.device);
            StreamWorkspace& w = st.ws[prob.stream];
            const size_t bytes = static_cast<size_t>(ga + gw) * 32 * kblocks;
            bool usable        = w.relaid_bytes >= bytes;
            if(!usable)
            {
                cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
                cudaStreamIsCapturing(prob.stream, &cap);
                if(cap == cudaStreamCaptureStatusNone)
                {
                    retire(st, w.relaid);
                    w.relaid       = nullptr;
                    w.relaid_bytes = 0;
                    B200_CUDA(cudaMalloc(&w.relaid, bytes));
                    w.relaid_bytes = bytes;
                    usable         = true;
                }
            }
            if(usable)
            {
                relaid = static_cast<uint32_t*>(w.relaid);
                auto run = [&](const ScaleOperand& sf, uint32_t* dst, long long groups) {
                    const long long total = groups * (kblocks / 4) * 32;
                    const int blocks      = static_cast<int>(std::min<long long>((total + 255) / 256, 148LL * 16));
                    relay_e8m0_shuffle_kernel<<<blocks, 256, 0, prob.stream>>>(static_cast<const uint8_t*>(sf.ptr), dst, static_cast<int>(groups),
                                                                               static_cast<int>(sf.padded_cols), kblocks);
                    B200_CUDA(cudaGetLastError());
                    g_launches.fetch_add(1);
                };
                run(prob.act_sf, relaid, ga);
                run(prob.wgt_sf, relaid + ga * 32 * (kblocks / 4), gw);
            }
        }
        if(relaid != nullptr)
        {
            GemmProblem p2 = prob;
            p2.act_sf      = ScaleOperand{relaid, SFW_G1250, ga * 32, kblocks};
            p2.wgt_sf      = ScaleOperand{relaid + ga * 32 * (kblocks / 4), SFW_G1250, gw * 32, kblocks};
            launch_gemm_locked(p2);
            return;
        }
    }

    if(prob.kind == PK_MXF8F4 && prob.M >= kWidenPrepassMinM && prob.scratch == nullptr && prob.wgt.mode == OPM_TILE16 &&
       prob.N % 16 == 0 && prob.K % 64 == 0 && !widen_prepass_disabled())
    {
        int prev_dev = 0;
        B200_CUDA(cudaGetDevice(&prev_dev));
        if(prev_dev != prob.device)
            B200_CUDA(cudaSetDevice(prob.device));
        struct Restore
        {
            int prev, cur;
            ~Restore()
            {
                if(prev != cur)
                    cudaSetDevice(prev);
            }
        } restore{prev_dev, prob.device};
        void* widened = nullptr;
        {
            std::lock_guard<std::mutex> lk(g_mutex);
            DeviceState& st    = device_state(prob.device);
            StreamWorkspace& w = st.ws[prob.stream];
            const size_t bytes = static_cast<size_t>(prob.N) * static_cast<size_t>(prob.K);
            bool usable        = w.widened_bytes >= bytes;
            if(!usable)
            {
                cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
                cudaStreamIsCapturing(prob.stream, &cap);
                if(cap == cudaStreamCaptureStatusNone)
                {
                    retire(st, w.widened);
                    w.widened       = nullptr;
                    w.widened_bytes = 0;
                    B200_CUDA(cudaMalloc(&w.widened, bytes));
                    w.widened_bytes = bytes;
                    usable          = true;
                }
            }
            if(usable)
            {
                widened                 = w.widened;
                const int chunks_in     = static_cast<int>(prob.K / 2 / 16);
                const long long rblocks = prob.N / 16;
                const long long total   = rblocks * chunks_in * 16;
                const int threads       = 256;
                const int blocks        = static_cast<int>(std::min<long long>((total + threads - 1) / threads, 148LL * 16));
                widen_e2m1_tile16_kernel<<<blocks, threads, 0, prob.stream>>>(static_cast<const uint4*>(prob.wgt.ptr),
                                                                              static_cast<uint4*>(widened), rblocks, chunks_in);
                B200_CUDA(cudaGetLastError());
                g_launches.fetch_add(1);
            }
        }
        if(widened != nullptr)
        {
            GemmProblem p2 = prob;
            p2.kind        = PK_MXFP8;
            p2.wgt.ptr     = widened;
            p2.wgt.kbytes  = prob.K;
            p2.wgt.ld_bytes = prob.K;
            launch_gemm_locked(p2);
            return;
        }
    }
    launch_gemm_locked(prob);
}

static void launch_gemm_locked(const GemmProblem& prob)
{
    B200_CHECK(prob.M > 0 && prob.N > 0 && prob.K > 0, "empty GEMM: M=", prob.M, " N=", prob.N, " K=", prob.K);
    B200_CHECK(prob.M < (1LL << 31) && prob.N < (1LL << 31) && prob.K < (1LL << 31), "dimension too large");
    const int kkind = kernel_kind_of(prob.kind);

    int prev_dev = 0;
    B200_CUDA(cudaGetDevice(&prev_dev));
    if(prev_dev != prob.device)
        B200_CUDA(cudaSetDevice(prob.device));
    struct Restore
    {
        int prev, cur;
        ~Restore()
        {
            if(prev != cur)
                cudaSetDevice(prev);
        }
    } restore{prev_dev, prob.device};

    std::lock_guard<std::mutex> lk(g_mutex);
    // With caller-provided scratch nothing may be allocated: the device facts come from attribute queries and
    // the library's own per-device record (which owns a cudaMalloc'ed status buffer) is left alone.
    DeviceState local_state;
    if(prob.scratch != nullptr)
    {
        B200_CUDA(cudaDeviceGetAttribute(&local_state.sm_count, cudaDevAttrMultiProcessorCount, prob.device));
        B200_CUDA(cudaDeviceGetAttribute(&local_state.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, prob.device));
        int cc_major = 0;
        B200_CUDA(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, prob.device));
        B200_CHECK(cc_major == 10, "this library only runs on sm_100 class GPUs");
        local_state.status = prob.scratch->status;
    }
    DeviceState& st = (prob.scratch != nullptr) ? local_state : device_state(prob.device);
    require_healthy(st, prob.device);

    KernelConfig cfg = prob.cfg;
    const bool requant = (prob.out_mode == OUT_E2M1 || prob.out_mode == OUT_MXFP8);
    if(requant)
    {
        // the re-quantising epilogue owns whole 128-column blocks of a row: activations on the 128-row slot, no K split,
        // tile width 128 or 256
        B200_CHECK(prob.kind == PK_MXFP4 || prob.kind == PK_NVFP4, "low-precision outputs are built for the MXFP4 / NVFP4 GEMM only");
        B200_CHECK(prob.N % 128 == 0, "low-precision outputs need N % 128 == 0 (got N=", prob.N, ")");
        B200_CHECK(prob.out_mode != OUT_MXFP8 || (prob.M % 64 == 0 && prob.out_scale != nullptr), "the mxfp8 output needs M % 64 == 0 and an out_scale tensor");
        B200_CHECK(prob.bias == nullptr, "low-precision outputs take no bias");
        cfg.swap        = 0;
        cfg.log2_splitk = 0;
        if(cfg.bn != 128 && cfg.bn != 256)
            cfg.bn = (prob.N % 256 == 0 && prob.M > 256) ? 256 : 128;
    }
    B200_CHECK(prob.batch == 1 || (prob.kind == PK_BF16 && prob.act.mode == OPM_BATCHED && prob.wgt.mode == OPM_BATCHED),
               "internal: batched launches are built for row-major bf16 operands");
    choose_config(prob.kind, prob.M, prob.N, prob.K, st.sm_count, cfg);
    B200_CHECK(cfg.log2_splitk >= 0 && cfg.log2_splitk <= 8, "log2 of the K split must be between 0 and 8 (got ", cfg.log2_splitk, ")");
    {
        bool ok = false;
        for(int b : kBnMenu)
            ok |= (b == cfg.bn);
        B200_CHECK(ok, "unsupported tile width ", cfg.bn);
    }
    const int cg = cfg.cg;
    B200_CHECK(cg == 1 || cg == 2, "internal: CTAs per tile");
    if(try_launch_decode(prob, cfg, kkind, st))
        return;
    B200_CHECK(cg == 1 || cfg.bn % 32 == 0, "a CTA-pair tile needs a width that is a multiple of 32");
    const Operand& P       = cfg.swap ? prob.wgt : prob.act;
    const Operand& Q       = cfg.swap ? prob.act : prob.wgt;
    const ScaleOperand& SP = cfg.swap ? prob.wgt_sf : prob.act_sf;
    const ScaleOperand& SQ = cfg.swap ? prob.act_sf : prob.wgt_sf;
    const bool mixed     = (kkind == KIND_MXF8F4);
    const int f4_operand = mixed ? (cfg.swap ? 1 : 2) : 0; // the weight is the packed e2m1 operand
    if(mixed)
        B200_CHECK(prob.act.kbytes == 2 * prob.wgt.kbytes && prob.wgt.mode == OPM_TILE16,
                   "mixed MXFP8 x MXFP4: the weight must be packed e2m1 in the 16x16-byte tiled layout");
    else
        B200_CHECK(P.kbytes == Q.kbytes, "operands disagree on K bytes: ", P.kbytes, " vs ", Q.kbytes);
    B200_CHECK(cfg.bn % 32 == 0 || Q.rows <= cfg.bn, "a tile width of ", cfg.bn,
               " only serves problems with at most that many rows on that side");

    const int num_k_iters = static_cast<int>((prob.act.kbytes + kTileKBytes - 1) / kTileKBytes);
    int splits            = 1 << cfg.log2_splitk;
    while(splits > num_k_iters)
        splits >>= 1;
    B200_CHECK(static_cast<long long>(num_k_iters) * (splits + 1) < (1LL << 31), "K x split count too large");
    const int atoms_k  = (kkind == KIND_NVF4) ? 4 : ((kkind == KIND_MXF4) ? 2 : 1);
    const int sf_cols  = sf_cols_per_stage(kkind);
    const int sf_unit  = sf_unit_of(kkind);
    // the output leaves through shared memory and TMA tile stores when its pitch and base allow a tensor map
    const bool tma_store = ((reinterpret_cast<uintptr_t>(prob.out) & 15) == 0) && (prob.ldo % 8 == 0) && (cfg.swap || cfg.bn >= 32) &&
                           (prob.out_mode == OUT_BF16 || prob.out_mode == OUT_F16) && prob.batch == 1;
    // Decode shapes: the K split runs across the CTAs of a thread-block cluster, one output tile per cluster; the
    // partial accumulators meet in the first CTA's shared memory instead of a global workspace.
    int csplit = 1;
    // (only with the weights on the 128-row slot: for row-major tiles, whose partial tiles are wide, it was measured two to
    // five times slower than the workspace split)
    if(cfg.swap && cg == 1 && splits > 1 && splits <= 8 && prob.scratch == nullptr && !cluster_split_disabled() &&
       max_stages(cfg.bn, cg, st.smem_optin, f4_operand, sf_unit, tma_store, splits) >= 4)
    {
        csplit = splits;
        splits = 1;
    }
    const int max_st = max_stages(cfg.bn, cg, st.smem_optin, f4_operand, sf_unit, tma_store, csplit);
    B200_CHECK(max_st >= 2, "tile ", 128 * cg, "x", cfg.bn, " does not fit in shared memory");
    int stages = cfg.stages <= 0 ? max_st : std::min(cfg.stages, max_st);

    const int tile_rows_p = kTileP * cg;
    const int tiles_p = static_cast<int>((P.rows + tile_rows_p - 1) / tile_rows_p);
    const int tiles_q = static_cast<int>((Q.rows + cfg.bn - 1) / cfg.bn);
    B200_CHECK(tiles_q <= 65535 && splits <= 65535, "grid too large");
    const int counter_slots = (prob.scratch != nullptr) ? prob.scratch->counter_slots : kCounterSlots;
    B200_CHECK(splits == 1 || static_cast<long long>(tiles_p) * tiles_q * cg * prob.batch <= counter_slots,
               "split-K supports at most ", counter_slots, " output tiles here");
    B200_CHECK(static_cast<long long>(tiles_p) * tiles_q * prob.batch * std::max(splits, 1) < (1LL << 31), "too many work units");

    unsigned long long* trace = nullptr;
#ifdef AITER_B200_TRACING
    static const bool trace_on = (std::getenv("AITER_B200_TRACE") != nullptr);
    // AITER_B200_TRACE_EVERY=n: every launch stamps, only every n-th is fetched and printed, and nothing is cleared
    // in between, so that the printed launch ran back to back with its predecessors
    static const int trace_every = std::getenv("AITER_B200_TRACE_EVERY") ? std::atoi(std::getenv("AITER_B200_TRACE_EVERY")) : 1;
    static int trace_seq = 0;
    bool trace_print = false;
    if(trace_on && prob.scratch == nullptr)
    {
        if(st.trace == nullptr)
        {
            B200_CUDA(cudaMalloc(&st.trace, kTraceWords * sizeof(unsigned long long)));
            B200_CUDA(cudaMemset(st.trace, 0, kTraceWords * sizeof(unsigned long long)));
        }
        if(trace_every <= 1)
            B200_CUDA(cudaMemsetAsync(st.trace, 0, kTraceWords * sizeof(unsigned long long), prob.stream));
        trace       = st.trace;
        trace_print = (trace_every <= 1) || (++trace_seq % trace_every == 0);
    }
#endif

    float* ws_partial        = nullptr;
    unsigned int* ws_counter = nullptr;
    if(splits > 1)
    {
        const size_t bytes = static_cast<size_t>(prob.batch) * tiles_p * tiles_q * cg * splits * static_cast<size_t>(cfg.bn) * kTileP * sizeof(float);
        if(prob.scratch != nullptr)
        {
            B200_CHECK(bytes <= prob.scratch->partial_bytes, "this shape needs ", bytes, " bytes of split-K scratch, more than the ",
                       prob.scratch->partial_bytes, " bytes of static scratch this entry point owns");
            ws_partial = prob.scratch->partial;
            ws_counter = prob.scratch->counter;
        }
        else
        {
            StreamWorkspace& w = stream_workspace(st, prob.stream, bytes);
            ws_partial         = w.partial;
            ws_counter         = w.counter;
        }
    }

    // tensor maps: every CTA stages 128 rows of P and bn / cg rows of Q per K tile
    CUtensorMap mp  = operand_map(P, kTileP, cfg.swap ? "weight operand" : "activation operand", f4_operand == 1 ? 64 : kTileKBytes);
    CUtensorMap mq  = operand_map(Q, cfg.bn / cg, cfg.swap ? "activation operand" : "weight operand", f4_operand == 2 ? 64 : kTileKBytes);
    CUtensorMap msp = mp, msq = mq;
    int sfw = SFW_NONE;
    const int kblocks = static_cast<int>(prob.K / 32);
    if(kkind != KIND_BF16)
    {
        B200_CHECK(SP.wire == SQ.wire && SP.wire != SFW_NONE, "both scale tensors must use the same wire layout");
        sfw = SP.wire;
        const int chunk = (sfw == SFW_E8M0_SHUFFLE) ? 256 : 128 * atoms_k;
        msp = scale_map(SP, chunk, 4, cfg.swap ? "weight scales" : "activation scales");
        msq = scale_map(SQ, chunk, (cfg.bn + 31) / 32, cfg.swap ? "activation scales" : "weight scales");
        B200_CHECK(sfw != SFW_E8M0_SHUFFLE || kkind == KIND_MXF4, "the e8m0_shuffle scale layout is only wired for MXFP4");
        B200_CHECK(kkind != KIND_NVF4 || sfw == SFW_G1250, "NVFP4 scales arrive in tiles of 32 rows x 8 scales");
        const long long need_cols = (kkind == KIND_NVF4) ? prob.K / 16 : (sfw == SFW_E8M0_SHUFFLE) ? (kblocks + 7) / 8 * 8 : kblocks;
        B200_CHECK(SP.padded_cols >= need_cols && SQ.padded_cols >= need_cols, "scale tensors have too few columns: need ",
                   need_cols, ", got ", SP.padded_cols, " and ", SQ.padded_cols);
        B200_CHECK(SP.padded_rows % 32 == 0 && SQ.padded_rows % 32 == 0, "scale rows must be padded to a multiple of 32");
        B200_CHECK(SP.padded_rows >= (P.rows + 31) / 32 * 32 && SQ.padded_rows >= (Q.rows + 31) / 32 * 32,
                   "scale tensors have too few rows");
        B200_CHECK(((reinterpret_cast<uintptr_t>(SP.ptr) | reinterpret_cast<uintptr_t>(SQ.ptr)) & 3) == 0,
                   "scale tensors must be 4-byte aligned");
        if(sfw == SFW_G1250)
            B200_CHECK(prob.K % (kkind == KIND_MXF8 || kkind == KIND_MXF8F4 ? 128 : 256) == 0, "K must be a multiple of ",
                       (kkind == KIND_MXF8 || kkind == KIND_MXF8F4 ? 128 : 256), " for this scale layout");
    }

    PersistentParams prm{};
    prm.rows_p         = static_cast<int>(P.rows);
    prm.rows_q         = static_cast<int>(Q.rows);
    prm.num_k_iters    = num_k_iters;
    prm.kblocks        = kblocks;
    prm.bn             = cfg.bn;
    prm.p_mode         = P.mode;
    prm.q_mode         = Q.mode;
    prm.f4_operand     = f4_operand;
    prm.transposed_out = cfg.swap;
    prm.tiles_p        = tiles_p;
    prm.tiles_q        = tiles_q;
    prm.splits         = splits;
    prm.sfp            = static_cast<const uint32_t*>(SP.ptr);
    prm.sfq            = static_cast<const uint32_t*>(SQ.ptr);
    prm.sfp_groups     = static_cast<int>(SP.padded_rows / 32);
    prm.sfq_groups     = static_cast<int>(SQ.padded_rows / 32);
    prm.sfp_row_words  = static_cast<int>(SP.padded_cols * 8);
    prm.sfq_row_words  = static_cast<int>(SQ.padded_cols * 8);
    prm.out            = prob.out;
    prm.ldo            = prob.ldo;
    prm.out_mode       = prob.out_mode;
    prm.out_scale      = static_cast<uint8_t*>(prob.out_scale);
    prm.out_scale_cols = static_cast<int>(prob.N / 128);
    prm.noscale        = prob.noscale;
    prm.batch          = static_cast<int>(prob.batch);
    prm.out_batch_stride  = prob.out_batch_stride;
    prm.bias_batch_stride = prob.bias_batch_stride;
    prm.bias           = prob.bias;
    prm.bias_is_bf16   = prob.bias_is_bf16;
    prm.bias_on_q      = cfg.swap ? 0 : 1;
    prm.alpha          = prob.alpha;
    prm.beta           = prob.beta;
    prm.status         = st.status;
    prm.trace          = trace;
    prm.ws_partial     = ws_partial;
    prm.ws_counter     = ws_counter;
    // TMEM: n_acc accumulators of acc_stride columns, then one scale buffer per shared-memory stage
    prm.acc_stride = (cfg.bn + 31) & ~31;
    prm.sf_cols    = sf_cols;
    prm.csplit            = csplit;
    {
        const int ksplit = csplit > 1 ? csplit : splits;
        int sh           = 0;
        while((1 << sh) < ksplit)
            ++sh;
        prm.split_shift = ((1 << sh) == ksplit) ? sh : -1;
    }
    const long long units = static_cast<long long>(prob.batch) * tiles_p * tiles_q * splits;
    // a cluster-split tile owns its cluster for the whole launch: one cluster per tile, however many run at once
    const int clusters    = csplit > 1 ? static_cast<int>(units) : static_cast<int>(std::min<long long>(units, st.sm_count / cg));
    const bool multi_unit = units > clusters;
    prm.n_acc = (multi_unit && 2 * prm.acc_stride + 2 * sf_cols <= 512) ? 2 : 1;
    while(prm.n_acc * prm.acc_stride + stages * sf_cols > 512 && stages > 2)
        --stages;
    B200_CHECK(prm.n_acc * prm.acc_stride + stages * sf_cols <= 512, "internal: TMEM budget exceeded");
    prm.stages       = stages;
    prm.sf_tmem_base = prm.n_acc * prm.acc_stride;
    int cols         = 32;
    while(cols < prm.sf_tmem_base + stages * sf_cols)
        cols <<= 1;
    prm.tmem_cols = cols;
    // 2: 64 columns per store (row-major output, tile width a multiple of 64, no K split); 1: 32 per store
    const bool wide_store  = tma_store && !cfg.swap && cfg.bn % 64 == 0 && splits == 1;
    prm.tma_store          = tma_store ? (wide_store ? 2 : 1) : 0;
    // the wide stores get a second staging buffer where that costs no pipeline stage
    prm.epi_bufs = tma_store ? 1 : 0;
    if(wide_store && static_cast<int>(make_persistent_smem(cfg.bn, cg, stages, f4_operand, sf_unit, 2, csplit).total) + 1024 <= st.smem_optin)
        prm.epi_bufs = 2;
    const PersistentSmem L = make_persistent_smem(cfg.bn, cg, stages, f4_operand, sf_unit, prm.epi_bufs, csplit);
    const size_t smem      = L.total + 1024;
    // Tile order.  When the Q operand (the weights of a tall problem) is much larger than what L2 keeps beside the
    // streaming P operand and the output, walk it in panels of about 32 MB.
    prm.panel_q = 0;
    {
        const double q_tile_bytes = static_cast<double>(cfg.bn) * static_cast<double>(Q.kbytes);
        const double q_bytes      = q_tile_bytes * tiles_q;
        if(!cfg.swap && csplit == 1 && tiles_q > 1 && q_bytes > 48e6 && !panel_order_disabled())
        {
            const int w0     = std::max(1, static_cast<int>(32e6 / q_tile_bytes));
            const int panels = (tiles_q + w0 - 1) / w0;
            const int w      = (tiles_q + panels - 1) / panels; // equal panels
            if(w < tiles_q)
                prm.panel_q = w;
        }
    }
    CUtensorMap mo         = mp;
    if(tma_store)
    {
        // bf16 [M][N] seen as bytes; one box = 32 values of the fast dimension by 32 rows (or the tile's chunk of rows
        // when the 128-row slot holds the weights and the store is transposed)
        const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(prob.N) * 2, static_cast<cuuint64_t>(prob.M)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(prob.ldo) * 2};
        const cuuint32_t box[2]     = {wide_store ? 128u : 64u, static_cast<cuuint32_t>(cfg.swap ? (cfg.bn < 32 ? 16 : 32) : 32)};
        mo = encode_map(prob.out, 2, dims, strides, box,
                        cfg.swap ? CU_TENSOR_MAP_SWIZZLE_NONE : (wide_store ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B), "output");
    }
    const int ctas         = clusters * cg * csplit;
    if(kkind == KIND_BF16)
        launch_persistent_cg<KIND_BF16, SFW_NONE>(cg, ctas, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_MXF8 && sfw == SFW_G1250)
        launch_persistent_cg<KIND_MXF8, SFW_G1250>(cg, ctas, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_MXF4 && sfw == SFW_E8M0_SHUFFLE)
        launch_persistent_cg<KIND_MXF4, SFW_E8M0_SHUFFLE>(cg, ctas, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_MXF4 && sfw == SFW_G1250)
        launch_persistent_cg<KIND_MXF4, SFW_G1250>(cg, ctas, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_MXF8F4 && sfw == SFW_G1250)
        launch_persistent_cg<KIND_MXF8F4, SFW_G1250>(cg, ctas, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else if(kkind == KIND_NVF4 && sfw == SFW_G1250)
        launch_persistent_cg<KIND_NVF4, SFW_G1250>(cg, ctas, smem, prob.stream, mp, mq, msp, msq, mo, prm);
    else
        fail("no kernel instance for kind ", kkind, " with scale layout ", sfw);

#ifdef AITER_B200_TRACING
    if(trace != nullptr && trace_print)
        print_trace(st, prob, cfg, tiles_p, tiles_q, splits, stages);
#endif
}

// One UE8M0 byte per (row, 128-wide K block) -> the (m/32, k/4, 32, 4) order of the MXFP8 kernel: the four 32-blocks
// of a 128 block share the byte.  rows_per_scale = 1 (activations) or 128 (weights: one byte per 128 x 128 block).
__global__ void expand_block128_scales_kernel(const uint8_t* __restrict__ src, long long stride_row, long long stride_k, uint32_t* __restrict__ dst,
                                              long long rows, long long groups, int kb128, int rows_per_scale)
{
    const long long total = groups * kb128 * 32;
    for(long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
        i += static_cast<long long>(gridDim.x) * blockDim.x)
    {
        const int r         = static_cast<int>(i & 31);
        const long long t   = i >> 5;
        const int kb        = static_cast<int>(t % kb128);
        const long long row = (t / kb128) * 32 + r;
        const uint32_t b    = row < rows ? src[(row / rows_per_scale) * stride_row + kb * stride_k] : 0x7Fu;
        dst[i]              = b * 0x01010101u;
    }
}

static void launch_blockscale_e8m0(const BlockScaleProblem& prob)
{
    int prev_dev = 0;
    B200_CUDA(cudaGetDevice(&prev_dev));
    if(prev_dev != prob.device)
        B200_CUDA(cudaSetDevice(prob.device));
    struct Restore
    {
        int prev, cur;
        ~Restore()
        {
            if(prev != cur)
                cudaSetDevice(prev);
        }
    } restore{prev_dev, prob.device};
    const int kb128    = static_cast<int>(prob.K / 128);
    const long long ga = (prob.M + 31) / 32, gw = (prob.N + 31) / 32;
    uint32_t* buf      = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mutex);
        DeviceState& st    = device_state(prob.device);
        StreamWorkspace& w = st.ws[prob.stream];
        const size_t bytes = static_cast<size_t>(ga + gw) * 32 * kb128 * 4;
        if(w.relaid_bytes < bytes)
        {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            cudaStreamIsCapturing(prob.stream, &cap);
            B200_CHECK(cap == cudaStreamCaptureStatusNone, "the scale buffer must grow (", bytes,
                       " bytes) but the stream is being captured; run this shape once outside capture first");
            retire(st, w.relaid);
            w.relaid       = nullptr;
            w.relaid_bytes = 0;
            B200_CUDA(cudaMalloc(&w.relaid, bytes));
            w.relaid_bytes = bytes;
        }
        buf = static_cast<uint32_t*>(w.relaid);
        auto run = [&](const uint8_t* src, long long sr, long long sk, uint32_t* dst, long long rows, long long groups, int per) {
            const long long total = groups * kb128 * 32;
            const int blocks      = static_cast<int>(std::min<long long>((total + 255) / 256, 148LL * 8));
            expand_block128_scales_kernel<<<blocks, 256, 0, prob.stream>>>(src, sr, sk, dst, rows, groups, kb128, per);
            B200_CUDA(cudaGetLastError());
            g_launches.fetch_add(1);
        };
        run(reinterpret_cast<const uint8_t*>(prob.x_scale), prob.xs_stride_m, prob.xs_stride_k, buf, prob.M, ga, 1);
        run(reinterpret_cast<const uint8_t*>(prob.w_scale), kb128, 1, buf + ga * 32 * kb128, prob.N, gw, 128);
    }
    GemmProblem p;
    p.kind   = PK_MXFP8;
    p.M = prob.M; p.N = prob.N; p.K = prob.K;
    p.act    = prob.act;
    p.wgt    = prob.wgt;
    p.act_sf = ScaleOperand{buf, SFW_G1250, ga * 32, prob.K / 32};
    p.wgt_sf = ScaleOperand{buf + ga * 32 * kb128, SFW_G1250, gw * 32, prob.K / 32};
    p.out      = prob.out;
    p.ldo      = prob.ldo;
    p.out_mode = prob.out_mode;
    p.device   = prob.device;
    p.stream   = prob.stream;
    p.cfg      = prob.cfg;
    launch_gemm(p);
}

static bool few_rows_disabled()
{
    static const bool off = (std::getenv("AITER_B200_NO_BLOCKSCALE_FEWROWS") != nullptr);
    return off;
}

// up to 64 activation rows (and a K whose unsplit scale table, 64 KB at most, fits beside the stages)
static bool use_few_rows(const BlockScaleProblem& prob)
{
    return prob.M <= 64 && prob.K <= 32768 && !few_rows_disabled();
}
// the same kernel also takes several tiles of 64 rows, each a CTA of its own on the same weight tile: up to four by the
// launcher's own rule (while all of them fit the machine at once), up to sixteen by name
static bool few_rows_can_serve(const BlockScaleProblem& prob, long long max_rows = 256)
{
    return prob.M <= max_rows && prob.K <= 32768 && !few_rows_disabled();
}

bool parse_blockscale_name(const char* name, int& variant, int& log2_splitk)
{
    if(name == nullptr || name[0] == 0)
        return false;
    static const struct { const char* base; int variant; } kNames[] = {{"bs_fewrows", 1}, {"bs_128x128", 2}, {"bs_256x256", 3}, {"bs_256x128", 4}};
    for(const auto& n : kNames)
    {
        const size_t len = std::strlen(n.base);
        if(std::strncmp(name, n.base, len) != 0)
            continue;
        int l2 = -1, more = 0;
        if(name[len] != 0 && (std::sscanf(name + len, "_k%d%n", &l2, &more) != 1 || name[len + more] != 0 || l2 < 0 || l2 > 4))
            return false;
        variant     = n.variant;
        log2_splitk = l2;
        return true;
    }
    return false;
}

void launch_blockscale(const BlockScaleProblem& prob)
{
    if(prob.M == 0 && prob.N > 0 && prob.K > 0)
        return;
    B200_CHECK(!(prob.scales_are_e8m0 && prob.variant > 1), "bs_128x128 / bs_256x256 / bs_256x128 take fp32 scales; e8m0 scales run on bs_fewrows or an MXFP8 kernel name");
    // (65..256 rows: tiles of 64 rows on the few-rows kernel while all of them fit the machine at once, as for fp32 scales)
    auto few_by_tiles = [&]() {
        return few_rows_can_serve(prob) && ((prob.N + kBsTileN - 1) / kBsTileN) * ((prob.M + 63) / 64) <= device_sm_count(prob.device);
    };
    if(prob.scales_are_e8m0 && prob.variant == 0 && (prob.cfg_given || !(use_few_rows(prob) || few_by_tiles())))
    {
        // powers of two ride the block-scaled MMA; few rows stay on the few-rows kernel below, which reads the
        // e8m0 bytes itself (one launch, no scale expansion pass: 128 x 4096 x 4096 18.6 -> 10.6 us)
        B200_CHECK(prob.K % 128 == 0, "K must be a multiple of 128 for 128-wide scale blocks (got ", prob.K, ")");
        launch_blockscale_e8m0(prob);
        return;
    }
    B200_CHECK(prob.M > 0 && prob.N > 0 && prob.K > 0, "empty GEMM: M=", prob.M, " N=", prob.N, " K=", prob.K);
    B200_CHECK(prob.K % 128 == 0, "K must be a multiple of 128 for 128-wide scale blocks (got ", prob.K, ")");
    int prev_dev = 0;
    B200_CUDA(cudaGetDevice(&prev_dev));
    if(prev_dev != prob.device)
        B200_CUDA(cudaSetDevice(prob.device));
    struct Restore
    {
        int prev, cur;
        ~Restore()
        {
            if(prev != cur)
                cudaSetDevice(prev);
        }
    } restore{prev_dev, prob.device};
    std::lock_guard<std::mutex> lk(g_mutex);
    DeviceState& st = device_state(prob.device);
    require_healthy(st, prob.device);

    BlockScaleParams prm{};
    prm.M           = static_cast<int>(prob.M);
    prm.N           = static_cast<int>(prob.N);
    prm.k_blocks    = static_cast<int>(prob.K / 128);
    prm.a_mode      = prob.act.mode;
    prm.b_mode      = prob.wgt.mode;
    prm.x_scale     = prob.x_scale;
    prm.xs_stride_m = prob.xs_stride_m;
    prm.xs_stride_k = prob.xs_stride_k;
    prm.w_scale     = prob.w_scale;
    prm.out         = prob.out;
    prm.ldo         = prob.ldo;
    prm.out_mode    = prob.out_mode;
    prm.status      = st.status;
    prm.scales_e8m0 = prob.scales_are_e8m0 ? 1 : 0;
    // 256 x 256 tiles on persistent CTA pairs or 128 x 128 tiles on single CTAs: whichever needs less time by rounds x
    // (cycles per K block x K blocks + cycles per tile), as measured: ~1050 + 4000 for a pair (the tile's rows leave under
    // the next tile's first K blocks), ~810 + 6300 for a single CTA (one tile per CTA: set-up, pipeline fill and the
    // stores are paid per tile).  Few tiles favour the single-CTA kernel (M = 300, N = K = 4096: 96 CTAs and 15.3 us
    // against 32 pairs and 29.6 us), many tiles the pairs.
    const long long tiles128 = ((prob.M + kTileP - 1) / kTileP) * ((prob.N + kBsTileN - 1) / kBsTileN);
    const long long pairs256 = ((prob.M + 2 * kTileP - 1) / (2 * kTileP)) * ((prob.N + 2 * kBsTileN - 1) / (2 * kBsTileN));
    const long long single_cost = (tiles128 + st.sm_count - 1) / st.sm_count * (prm.k_blocks * 810LL + 6300);
    const long long pair_cost   = (pairs256 + st.sm_count / 2 - 1) / (st.sm_count / 2) * (prm.k_blocks * 1050LL + 4000);
    B200_CHECK(prob.variant != 1 || few_rows_can_serve(prob, 1024), "bs_fewrows serves at most 1024 activation rows");
    B200_CHECK((prob.variant != 3 && prob.variant != 4) || prob.M > kTileP, "bs_256x256 / bs_256x128 need more than 128 activation rows");
    // 65..256 rows: tiles of 64 rows on the few-rows kernel while all of them fit the machine at once (measured against the
    // 128 x 128 kernel: 256 x 4096 x 4096 15.1 -> 13.3 us, 96 x 4096 x 4096 14.1 -> 10.4 us, 200 x 1536 x 7168 16.3 -> 13.5 us;
    // with more tiles than SMs it loses: 256 x 7168 x 2048 10.7 -> 15.7 us)
    const long long few_tiles = ((prob.N + kBsTileN - 1) / kBsTileN) * ((prob.M + 63) / 64);
    const bool want_few  = prob.variant == 1 || (prob.variant == 0 && (use_few_rows(prob) || (few_rows_can_serve(prob) && few_tiles <= st.sm_count)));
    const bool want_pair = prob.variant == 3 || (prob.variant == 0 && !want_few && prob.M > kTileP && pair_cost < single_cost);
    const int forced_splits = prob.log2_splitk >= 0 ? (1 << prob.log2_splitk) : 0; // 0: the cost model below decides
    if(prob.variant == 4)
    {
        // 256 x 128 tiles on CTA pairs
        const int stage_bytes = (kTileP + kBsPairNarrowN / 2) * kTileKBytes;
        int stages            = std::min((st.smem_optin - 2048) / stage_bytes, kMaxStages);
        stages                = std::max(2, std::min(stages, prm.k_blocks));
        prm.stages            = stages;
        const size_t smem     = static_cast<size_t>(stage_bytes) * stages + 512 + 1024;
        CUtensorMap ma = operand_map(prob.act, kTileP, "activation operand");
        CUtensorMap mb = operand_map(prob.wgt, kBsPairNarrowN / 2, "weight operand");
        static bool attr_done[64] = {};
        raise_smem_limit(gemm_a8w8_blockscale_pair_narrow_kernel, attr_done);
        prm.splits             = 1;
        const unsigned pairs_m = static_cast<unsigned>((prob.M + 2 * kTileP - 1) / (2 * kTileP));
        const unsigned tiles_n = static_cast<unsigned>((prob.N + kBsPairNarrowN - 1) / kBsPairNarrowN);
        B200_CHECK(tiles_n <= 65535, "N too large");
        cudaLaunchConfig_t lc{};
        lc.gridDim          = dim3(pairs_m * 2, tiles_n, 1);
        lc.blockDim         = dim3(kBlockScalePairThreads, 1, 1);
        lc.dynamicSmemBytes = smem;
        lc.stream           = prob.stream;
        cudaLaunchAttribute attr[2];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs    = attr;
        lc.numAttrs = pdl_disabled() ? 1 : 2;
        B200_CUDA(cudaLaunchKernelEx(&lc, gemm_a8w8_blockscale_pair_narrow_kernel, ma, mb, prm));
    }
    else if(want_pair)
    {
        // 256 x 256 tiles on CTA pairs
        const int stage_bytes = 2 * kTileP * kTileKBytes;
        const int epi_bytes   = 8 * 4096; // one output staging buffer per promotion warp
        int stages            = std::min((st.smem_optin - 2048 - epi_bytes) / stage_bytes, kMaxStages);
        stages                = std::max(2, std::min(stages, prm.k_blocks));
        prm.stages            = stages;
        const size_t smem     = static_cast<size_t>(stage_bytes) * stages + epi_bytes + 512 + 1024;
        CUtensorMap ma = operand_map(prob.act, kTileP, "activation operand");
        CUtensorMap mb = operand_map(prob.wgt, kTileP, "weight operand");
        // 16-bit outputs leave as warp-wide TMA tiles of 32 rows x 64 columns (bytes; 128-byte swizzle)
        CUtensorMap mo = ma;
        prm.tma_out    = 0;
        if((reinterpret_cast<uintptr_t>(prob.out) & 15) == 0 && prob.ldo % 8 == 0 && prob.out_mode != OUT_F32)
        {
            prm.tma_out                 = 64;
            const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(prob.N) * 2, static_cast<cuuint64_t>(prob.M)};
            const cuuint64_t strides[1] = {static_cast<cuuint64_t>(prob.ldo) * 2};
            const cuuint32_t box[2]     = {128u, 32u};
            mo = encode_map(prob.out, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "output");
        }
        static bool attr_done[64] = {};
        raise_smem_limit(gemm_a8w8_blockscale_pair_kernel, attr_done);
        prm.splits             = 1;
        // persistent: one CTA pair per two SMs (or per tile, if there are fewer), each walking tiles pair, pair + pairs, ...
        const long long pairs_m = (prob.M + 2 * kTileP - 1) / (2 * kTileP);
        const long long tiles_n = (prob.N + kBsPairN - 1) / kBsPairN;
        B200_CHECK(pairs_m * tiles_n < (1LL << 30), "too many output tiles");
        prm.pairs_m = static_cast<int>(pairs_m);
        prm.tiles_n = static_cast<int>(tiles_n);
        const unsigned clusters = static_cast<unsigned>(std::min<long long>(pairs_m * tiles_n, std::max(st.sm_count / 2, 1)));
        cudaLaunchConfig_t lc{};
        lc.gridDim          = dim3(clusters * 2, 1, 1);
        lc.blockDim         = dim3(kBlockScalePairThreads, 1, 1);
        lc.dynamicSmemBytes = smem;
        lc.stream           = prob.stream;
        cudaLaunchAttribute attr[2];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs    = attr;
        lc.numAttrs = pdl_disabled() ? 1 : 2;
        B200_CUDA(cudaLaunchKernelEx(&lc, gemm_a8w8_blockscale_pair_kernel, ma, mb, mo, prm));
    }
    else if(want_few)
    {
        // few activation rows: weights on the M side of the MMA, activations on its N side
        const int xr          = prob.M <= 16 ? 16 : (prob.M <= 32 ? 32 : 64);
        const int stage_bytes = (kBsTileN + xr) * kTileKBytes;
        CUtensorMap ma = operand_map(prob.act, xr, "activation operand");
        CUtensorMap mb = operand_map(prob.wgt, kBsTileN, "weight operand");
        dim3 grid(static_cast<unsigned>((prob.N + kBsTileN - 1) / kBsTileN), static_cast<unsigned>((prob.M + xr - 1) / xr), 1);
        const long long tiles = static_cast<long long>(grid.x) * grid.y;
        // split K across CTAs while the grid under-fills the machine and every slice keeps two K blocks; up to eight
        // slices of 16 or 32 rows form one cluster and meet in shared memory, the rest goes through the workspace
        static const bool no_split   = (std::getenv("AITER_B200_NO_BLOCKSCALE_SPLIT") != nullptr);
        static const bool no_cluster = (std::getenv("AITER_B200_NO_CLUSTER_SPLIT") != nullptr);
        const bool may_cluster       = !no_cluster;
        int splits = 1;
        while(!no_split && splits < (may_cluster ? 8 : 16) && tiles * (splits * 2) <= st.sm_count &&
              prm.k_blocks / (splits * 2) >= 2)
            splits *= 2;
        if(forced_splits > 0)
            splits = std::max(1, std::min(std::min(forced_splits, may_cluster ? 8 : 16), prm.k_blocks));
        prm.cluster = (may_cluster && splits > 1) ? 1 : 0;
        if(prm.cluster)
            ; // nothing to reserve: the slices meet in the reducing CTA's shared memory
        else if(splits > 1 && tiles <= kCounterSlots)
        {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            cudaStreamIsCapturing(prob.stream, &cap);
            const size_t bytes  = static_cast<size_t>(tiles) * splits * kBsTileN * xr * sizeof(float);
            StreamWorkspace& w0 = st.ws[prob.stream];
            if(cap != cudaStreamCaptureStatusNone && (w0.counter == nullptr || w0.partial_bytes < bytes))
                splits = 1; // the workspace may not grow inside a capture: run unsplit
            else
            {
                StreamWorkspace& w = stream_workspace(st, prob.stream, bytes);
                prm.ws_partial     = w.partial;
                prm.ws_counter     = w.counter;
            }
        }
        else
            splits = 1;
        prm.splits = splits;
        grid.z     = static_cast<unsigned>(splits);
        const int per_slice  = (prm.k_blocks + splits - 1) / splits;
        const int red_bytes  = prm.cluster ? (splits - 1) * (kBsTileN / splits) * xr * 4 : 0; // the other slices' share of this CTA's columns
        const int sc_bytes   = per_slice * xr * 4; // the slice's scale products
        prm.stages           = std::max(2, std::min(std::min((st.smem_optin - 2048 - red_bytes - sc_bytes) / stage_bytes, kMaxStages), per_slice));
        const size_t smem    = static_cast<size_t>(stage_bytes) * prm.stages + red_bytes + 512 + sc_bytes + 1024;
        cudaLaunchConfig_t lc{};
        lc.gridDim          = grid;
        lc.blockDim         = dim3(kFewRowsThreads, 1, 1);
        lc.dynamicSmemBytes = smem;
        lc.stream           = prob.stream;
        cudaLaunchAttribute attr[2];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = prm.cluster ? static_cast<unsigned>(splits) : 1u;
        attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs    = attr;
        lc.numAttrs = pdl_disabled() ? 1 : 2;
        // output as warp-wide TMA tiles: a warp owns 32 columns, or 16 when eight slices share the tile's 128
        CUtensorMap mo = ma;
        prm.tma_out    = 0;
        if((reinterpret_cast<uintptr_t>(prob.out) & 15) == 0 && prob.ldo % 8 == 0 && prob.out_mode != OUT_F32)
        {
            prm.tma_out                 = (prm.cluster && splits == 8) ? 16 : 32;
            const cuuint64_t dims[2]    = {static_cast<cuuint64_t>(prob.N) * 2, static_cast<cuuint64_t>(prob.M)};
            const cuuint64_t strides[1] = {static_cast<cuuint64_t>(prob.ldo) * 2};
            const cuuint32_t box[2]     = {static_cast<cuuint32_t>(prm.tma_out) * 2u, static_cast<cuuint32_t>(xr)};
            mo = encode_map(prob.out, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, "output");
        }
        static bool attr_done[3][64] = {};
        if(xr == 16)
        {
            raise_smem_limit(gemm_a8w8_blockscale_fewrows_kernel<16>, attr_done[0]);
            B200_CUDA(cudaLaunchKernelEx(&lc, gemm_a8w8_blockscale_fewrows_kernel<16>, ma, mb, mo, prm));
        }
        else if(xr == 32)
        {
            raise_smem_limit(gemm_a8w8_blockscale_fewrows_kernel<32>, attr_done[1]);
            B200_CUDA(cudaLaunchKernelEx(&lc, gemm_a8w8_blockscale_fewrows_kernel<32>, ma, mb, mo, prm));
        }
        else
        {
            raise_smem_limit(gemm_a8w8_blockscale_fewrows_kernel<64>, attr_done[2]);
            B200_CUDA(cudaLaunchKernelEx(&lc, gemm_a8w8_blockscale_fewrows_kernel<64>, ma, mb, mo, prm));
        }
        B200_CUDA(cudaGetLastError());
    }
    else
    {
        const int stage_bytes = (kTileP + kBsTileN) * kTileKBytes;
        int stages            = (st.smem_optin - 2048) / stage_bytes;
        stages                = std::min(stages, kMaxStages);
        stages                = std::max(2, std::min(stages, prm.k_blocks));
        prm.stages            = stages;
        const size_t smem     = static_cast<size_t>(stage_bytes) * stages + 512 + 1024;
        CUtensorMap ma = operand_map(prob.act, kTileP, "activation operand");
        CUtensorMap mb = operand_map(prob.wgt, kBsTileN, "weight operand");
        static bool attr_done[64] = {};
        raise_smem_limit(gemm_a8w8_blockscale_kernel, attr_done);
        dim3 grid(static_cast<unsigned>((prob.M + kTileP - 1) / kTileP), static_cast<unsigned>((prob.N + kBsTileN - 1) / kBsTileN), 1);
        B200_CHECK(grid.y <= 65535, "N too large");
        // few tiles (decode shapes): split K across CTAs while the grid under-fills the machine and every slice keeps
        // four K blocks; the slices meet in a per-stream fp32 workspace, the last to arrive reduces
        int splits = 1;
        const long long tiles = static_cast<long long>(grid.x) * grid.y;
        static const bool no_split = (std::getenv("AITER_B200_NO_BLOCKSCALE_SPLIT") != nullptr);
        while(!no_split && splits < 8 && tiles * (splits * 2) <= st.sm_count && prm.k_blocks / (splits * 2) >= 4)
            splits *= 2;
        if(forced_splits > 0)
            splits = std::max(1, std::min(std::min(forced_splits, 8), prm.k_blocks));
        if(splits > 1 && tiles <= kCounterSlots)
        {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            cudaStreamIsCapturing(prob.stream, &cap);
            const size_t bytes = static_cast<size_t>(tiles) * splits * kBsTileN * kTileP * sizeof(float);
            StreamWorkspace& w0 = st.ws[prob.stream];
            if(cap != cudaStreamCaptureStatusNone && (w0.counter == nullptr || w0.partial_bytes < bytes))
                splits = 1; // the workspace may not grow inside a capture: run unsplit
            else
            {
                StreamWorkspace& w = stream_workspace(st, prob.stream, bytes);
                prm.ws_partial     = w.partial;
                prm.ws_counter     = w.counter;
            }
        }
        else
            splits = 1;
        prm.splits = splits;
        grid.z     = static_cast<unsigned>(splits);
        {
            cudaLaunchConfig_t lc{};
            lc.gridDim          = grid;
            lc.blockDim         = dim3(kBlockScaleThreads, 1, 1);
            lc.dynamicSmemBytes = smem;
            lc.stream           = prob.stream;
            cudaLaunchAttribute attr[1];
            attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            lc.attrs    = attr;
            lc.numAttrs = pdl_disabled() ? 0 : 1;
            B200_CUDA(cudaLaunchKernelEx(&lc, gemm_a8w8_blockscale_kernel, ma, mb, prm));
        }
        B200_CUDA(cudaGetLastError());
    }
    g_launches.fetch_add(1);
}

} // namespace b200
