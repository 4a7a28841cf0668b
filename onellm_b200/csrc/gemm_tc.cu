// Context-phase projections (M > 64 tokens) on the 5th-generation tensor cores of sm_100a.
//
// Replaces the cuBLAS GEMM behind launchLinearGemm (src/kernels/qkv_linear.cu:8-65,
// src/kernels/cublas_wrapper.cc:45-90 of the reference) for prefill shapes: y[M,N] = x[M,K] . W with
// W [K,N] (the layer weights, N contiguous) or W [N,K] (the LM head), fp16 in, fp32 accumulate.
//
// Persistent: one block per SM walks 128 x 256 output tiles (with 128 x 128 tiles the operand traffic from L2
// into shared memory, 15.6 KB per MFLOP, was what bounded the kernel; the wider tile needs 11.7) in an order
// that keeps the tiles in flight on a near-square patch of the output.  Warp 0 streams 64-deep K slices of
// both operands into a ring of four shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte swizzle; no
// cluster multicast anywhere); one thread of warp 1 issues tcgen05.mma (M = 128, N = 256, K = 16, kind::f16)
// and releases each stage with tcgen05.commit; tensor memory holds two 256-column accumulators, so warps 2-5
// (tcgen05.ld, convert, store) drain tile i while the MMAs of tile i + 1 run.
// The [K,N] weight is used as it lies in memory: it is the "MN-major" B operand of the MMA
// (four 64-column TMA boxes per stage), so no transposed copy of the weights is ever made.
// Every wait on an mbarrier is bounded; on a time-out the block records it in a device flag,
// skips its stores, frees its tensor memory and exits.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "tc_common.cuh"

namespace onellm {

constexpr int kTcBM = 128, kTcBN = 256, kTcBK = 64;
constexpr int kTcStages = 4;
constexpr int kTcBand = 16;  // row tiles per band of the tile order
constexpr int kTcThreads = 192;      // producer warp, MMA warp, four epilogue warps
constexpr int kTcEpiThreads = 128;
constexpr int kTcATile = kTcBM * kTcBK * 2;        // 16 KB: 128 rows x 128 bytes
constexpr int kTcBTile = kTcBN * kTcBK * 2;        // 32 KB: [K,N] four boxes of 64 k-rows x 128 bytes; [N,K] 256 rows x 128 bytes
constexpr int kTcBChunk = 64 * kTcBK * 2;          // 8 KB: one 64-column chunk of a [K,N] stage
constexpr int kTcStageBytes = kTcATile + kTcBTile;
constexpr int kTcSmemBytes = kTcStages * kTcStageBytes + 1024 /* alignment slack */ + 256 /* barriers, TMEM address */;

// W_NK = false: W [K,N] (B operand MN-major);  W_NK = true: W [N,K] (B operand K-major).
// Persistent: grid = min(tiles, SMs) blocks of six warps; block c works on tiles c, c + grid, ... in band
// order (see below).  Warp 0 (one thread) is the TMA producer, warp 1 (one thread) issues the MMAs,
// warps 2-5 are the epilogue.  Tensor memory holds TWO 128 x 256 accumulators, so the MMAs of the next
// tile run while the epilogue warps drain the previous one.
// MODE 2: two [K,N] weights; the 256 accumulator columns of a tile are 128 columns of x.W (gate) beside the
// same 128 columns of x.W2 (up), and the epilogue stores silu(gate) * up: the gate GEMM, the up GEMM and
// launchAct of src/layers/ffn/ffn.cpp:62-66 in one pass, without the [T, 2, I] buffer.
// Epilogue options that let the context phase run without norm kernels, as the decode step does (the norm's gamma
// is multiplied into the weight rows beforehand):
//   row_ss:  sums of squares of the rows of x, as ss_parts partial sums per row; the result rows are scaled by
//            rsqrt(sum / K + eps), i.e. this is the projection of RMSNorm(x)
//   resid:   y = resid + bias + result (resid may be y itself: an element is read and written by the same thread)
//   ss_out:  [M, ceil(N / tile columns)]: the sum of squares of the stored (rounded) values of each row inside this
//            tile's columns -- the row_ss of the projection that reads y next.  Every entry is written by exactly
//            one block, so the sums do not depend on the order the blocks run in.
struct TcEpilogue {
    const float* row_ss;
    int ss_parts;
    float eps;
    const __half* resid;
    const __half* bias;
    float* ss_out;
};

template <int MODE>
__global__ void __launch_bounds__(kTcThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_b2, __half* y, int M, int N, int K, const TcEpilogue epi)
{
    constexpr bool W_NK = MODE == 1;
    constexpr bool DUAL = MODE == 2;
    constexpr int kOutN = DUAL ? kTcBN / 2 : kTcBN;  // output columns per tile
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment for the 128-byte swizzle pattern
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTcStages * kTcStageBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kTcStages + 4);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kTcStages);
    const uint32_t acc_full0 = smem_u32(bars + 2 * kTcStages), acc_empty0 = smem_u32(bars + 2 * kTcStages + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Tile order: the linear tile index walks down a band of kTcBand row tiles, then moves one column
    // tile to the right, so the tiles in flight at one time (one per SM) cover a near-square patch
    // of the output and share their A row blocks and B column blocks in L2.  (Row-major order made every
    // wave touch all column tiles of B: operands were read from DRAM seven times over.)
    const int tiles_m = (M + kTcBM - 1) / kTcBM, tiles_n = (N + kOutN - 1) / kOutN;
    const int n_tiles = tiles_m * tiles_n;
    auto tile_origin = [&](int t, int& m0, int& n0) {
        const int per_band = kTcBand * tiles_n;
        const int band = t / per_band, in_band = t % per_band;
        const int band_rows = min(kTcBand, tiles_m - band * kTcBand);
        m0 = (band * kTcBand + in_band % band_rows) * kTcBM;
        n0 = (in_band / band_rows) * kOutN;
    };
    const int k_steps = (K + kTcBK - 1) / kTcBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(acc_full0 + 8 * a, 1);
            mbar_init(acc_empty0 + 8 * a, kTcEpiThreads);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2u * kTcBN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    pdl_wait();  // x comes from the previous kernel in the stream

    if (warp == 0 && lane == 0) {
        // producer: one 64-deep slice of A and of B per stage, tile after tile
        int it = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            int m0, n0;
            tile_origin(t, m0, n0);
            for (int ks = 0; ks < k_steps; ks++, it++) {
                const int s = it % kTcStages;
                if (it >= kTcStages) ok = mbar_wait(empty0 + 8 * s, ((it / kTcStages) - 1) & 1);
                if (!ok) break;
                const uint32_t a_dst = smem_u32(smem + s * kTcStageBytes), b_dst = a_dst + kTcATile;
                mbar_expect_tx(full0 + 8 * s, kTcStageBytes);
                tma_load_2d(a_dst, &map_a, ks * kTcBK, m0, full0 + 8 * s);
                if (W_NK) {
                    tma_load_2d(b_dst, &map_b, ks * kTcBK, n0, full0 + 8 * s);
                } else if (DUAL) {
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        tma_load_2d(b_dst + c * kTcBChunk, &map_b, n0 + 64 * c, ks * kTcBK, full0 + 8 * s);
                        tma_load_2d(b_dst + (2 + c) * kTcBChunk, &map_b2, n0 + 64 * c, ks * kTcBK, full0 + 8 * s);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < kTcBN / 64; c++)
                        tma_load_2d(b_dst + c * kTcBChunk, &map_b, n0 + 64 * c, ks * kTcBK, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // instruction descriptor: D = f32, A = B = f16, A K-major, B MN-major unless W_NK, N = 256, M = 128
        const uint32_t idesc = (1u << 4) | ((W_NK ? 0u : 1u) << 16) | ((uint32_t)(kTcBN >> 3) << 17) | ((uint32_t)(kTcBM >> 4) << 24);
        int it = 0, lt = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, lt++) {
            const int acc = lt & 1, use = lt >> 1;
            // the accumulator must have been drained by the epilogue of the tile that used it before
            if (use >= 1) ok = mbar_wait(acc_empty0 + 8 * acc, (use - 1) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + (uint32_t)(acc * kTcBN);
            for (int ks = 0; ks < k_steps; ks++, it++) {
                const int s = it % kTcStages;
                ok = mbar_wait(full0 + 8 * s, (it / kTcStages) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(smem + s * kTcStageBytes), b_addr = a_addr + kTcATile;
#pragma unroll
                for (int kk = 0; kk < kTcBK / 16; kk++) {
                    // A: K-major, rows of 128 bytes, 8-row groups 1024 bytes apart; 16 k = 32 bytes further in the row
                    const uint64_t adesc = umma_desc(a_addr + kk * 32, 16, 1024);
                    // B [N,K]: same form.  B [K,N]: MN-major, 64-column chunks 8192 bytes apart (LBO), 8-row k groups
                    // 1024 bytes apart (SBO); 16 k = two groups further
                    const uint64_t bdesc = W_NK ? umma_desc(b_addr + kk * 32, 16, 1024) : umma_desc(b_addr + kk * 2048, kTcBChunk, 1024);
                    umma_f16(tmem_d, adesc, bdesc, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(empty0 + 8 * s);  // frees the stage when these MMAs have read it
            }
            if (ok) umma_commit(acc_full0 + 8 * acc);  // the tile is complete when everything issued so far has run
        }
        pdl_launch_dependents();
    } else if (warp >= 2) {
        // epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31, which are the tile rows of the same numbers
        const int q = warp & 3;
        int lt = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, lt++) {
            const int acc = lt & 1, use = lt >> 1;
            int m0, n0;
            tile_origin(t, m0, n0);
            ok = mbar_wait(acc_full0 + 8 * acc, use & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + q * 32 + lane;
            float inv = 1.f, sq = 0.f;
            if (epi.row_ss && row < M) {
                float ssum = 0.f;
                for (int pp = 0; pp < epi.ss_parts; pp++) ssum += epi.row_ss[(size_t)row * epi.ss_parts + pp];
                inv = rsqrtf(ssum / (float)K + epi.eps);
            }
#pragma unroll 1
            for (int c0 = 0; c0 < kOutN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kTcBN + c0), r);
                if (DUAL) {
                    uint32_t u[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kTcBN + kOutN + c0), u);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const float g = __uint_as_float(r[i]) * inv;
                        r[i] = __float_as_uint(g / (1.0f + __expf(-g)) * (__uint_as_float(u[i]) * inv));
                    }
                } else {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (epi.row_ss) {
#pragma unroll
                        for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * inv);
                    }
                }
                if (row < M) {
                    __half* dst = y + (size_t)row * N + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (n0 + c0 + 8 * j < N) {  // N is a multiple of 8
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) v[e] = __uint_as_float(r[8 * j + e]);
                            if (epi.resid) {
                                float a[8];
                                Vec16<__half>::load(epi.resid + (size_t)row * N + n0 + c0 + 8 * j, a);
#pragma unroll
                                for (int e = 0; e < 8; e++) v[e] += a[e];
                                if (epi.bias) {
                                    Vec16<__half>::load(epi.bias + n0 + c0 + 8 * j, a);
#pragma unroll
                                    for (int e = 0; e < 8; e++) v[e] += a[e];
                                }
                            }
                            const uint4 packed = Vec16<__half>::pack(v);
                            *reinterpret_cast<uint4*>(dst + 8 * j) = packed;
                            if (epi.ss_out) {
                                Vec16<__half>::unpack(packed, v);  // what the next projection will read
#pragma unroll
                                for (int e = 0; e < 8; e++) sq = fmaf(v[e], v[e], sq);
                            }
                        }
                    }
                }
            }
            if (epi.ss_out && row < M) epi.ss_out[(size_t)row * tiles_n + n0 / kOutN] = sq;
            // this thread's reads of the accumulator are over: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty0 + 8 * acc);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2u * kTcBN) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D fp16 tensor map: `inner` contiguous elements, `outer` rows of `inner` elements; box {64, box_outer}; 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint32_t box_outer)
{
    EncodeTiledFn enc = encode_tiled();
    ONELLM_REQUIRE(enc, ONELLM_ERR_CUDA, "gemm: cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * sizeof(__half)};
    const cuuint32_t box[2] = {64, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    ONELLM_REQUIRE(r == CUDA_SUCCESS, ONELLM_ERR_CUDA, "gemm: cuTensorMapEncodeTiled failed with %d", (int)r);
    return ONELLM_OK;
}

int gemm_f16_skinny(const __half* x, const __half* W, __half* y, int M, int N, int K, int w_layout, cudaStream_t st);

// mode 0: W [K,N]; 1: W [N,K]; 2: W and W2 [K,N], y = silu(x.W) * (x.W2)
static int gemm_tc_launch(const __half* x, const __half* W, const __half* W2, __half* y, int M, int N, int K, int mode, cudaStream_t st,
                          const TcEpilogue& epi = TcEpilogue{})
{
    ONELLM_REQUIRE(K % 8 == 0 && N % 8 == 0, ONELLM_ERR_UNSUPPORTED, "gemm: M > 64 needs K %% 8 == 0 and N %% 8 == 0 (K=%d N=%d)",
                   K, N);
    CUtensorMap map_a, map_b, map_b2;
    int rc = make_map(&map_a, x, (uint64_t)K, (uint64_t)M, kTcBM);
    if (rc) return rc;
    rc = mode == 1 ? make_map(&map_b, W, (uint64_t)K, (uint64_t)N, kTcBN) : make_map(&map_b, W, (uint64_t)N, (uint64_t)K, kTcBK);
    if (rc) return rc;
    map_b2 = map_b;
    if (mode == 2) {
        rc = make_map(&map_b2, W2, (uint64_t)N, (uint64_t)K, kTcBK);
        if (rc) return rc;
    }
    static DeviceOnce smem_attr[3];
    {
        const void* fn = mode == 0 ? (const void*)gemm_tc_kernel<0> : mode == 1 ? (const void*)gemm_tc_kernel<1> : (const void*)gemm_tc_kernel<2>;
        ONELLM_CUDA(smem_attr[mode].run([fn] { return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes); }));
    }
    const int out_n = mode == 2 ? kTcBN / 2 : kTcBN;
    const long tiles = (long)((N + out_n - 1) / out_n) * ((M + kTcBM - 1) / kTcBM);
    ONELLM_REQUIRE(tiles <= 0x7fffffffL, ONELLM_ERR_UNSUPPORTED, "gemm: too many tiles");
    const dim3 grid((unsigned)std::min<long>(tiles, num_sms()));  // persistent: one block per SM (shared memory allows no more)
    if (mode == 0)
        ONELLM_CUDA(launch_pdl(gemm_tc_kernel<0>, grid, dim3(kTcThreads), kTcSmemBytes, st, map_a, map_b, map_b2, y, M, N, K, epi));
    else if (mode == 1)
        ONELLM_CUDA(launch_pdl(gemm_tc_kernel<1>, grid, dim3(kTcThreads), kTcSmemBytes, st, map_a, map_b, map_b2, y, M, N, K, epi));
    else
        ONELLM_CUDA(launch_pdl(gemm_tc_kernel<2>, grid, dim3(kTcThreads), kTcSmemBytes, st, map_a, map_b, map_b2, y, M, N, K, epi));
    return ONELLM_OK;
}

int gemm_f16_large(const __half* x, const __half* W, __half* y, int M, int N, int K, int w_layout, cudaStream_t st)
{
    return gemm_tc_launch(x, W, nullptr, y, M, N, K, w_layout == ONELLM_W_NK ? 1 : 0, st);
}

// Gate and up projections with SwiGLU in the epilogue, M > 64.
int gemm_swiglu_f16_large(const __half* x, const __half* Wg, const __half* Wu, __half* out, int M, int I, int K, cudaStream_t st)
{
    return gemm_tc_launch(x, Wg, Wu, out, M, I, K, 2, st);
}

// Column tiles of a projection with N outputs (two weights: gate and up share a tile): the second extent of the
// [M, parts] array of partial row sums that onellm_gemm_rows writes.
int gemm_rows_parts(int N, bool dual)
{
    const int out_n = dual ? kTcBN / 2 : kTcBN;
    return (N + out_n - 1) / out_n;
}

// The large-M form of the norm-free projections (see TcEpilogue).
int gemm_rows_f16(const __half* x, const __half* W, const __half* W2, __half* y, int M, int N, int K, const float* row_ss, int ss_parts,
                  float eps, const __half* resid, const __half* bias, float* ss_out, cudaStream_t st)
{
    const TcEpilogue epi = {row_ss, ss_parts, eps, resid, resid ? bias : nullptr, ss_out};
    return gemm_tc_launch(x, W, W2, y, M, N, K, W2 ? 2 : 0, st, epi);
}

int attn_tc_timeout_flag();  // context_attn_tc.cu
int skinny_tc_flag();         // skinny_gemm_tc.cu

// 1 when a tensor-core block (projection or context attention) gave up a bounded wait since the last call.
int gemm_tc_timeout_flag()
{
    const int a = tc_flag_read_clear(), b = attn_tc_timeout_flag(), c = skinny_tc_flag();
    return (a < 0 || b < 0 || c < 0) ? -1 : (a | b | c);
}

}  // namespace onellm

extern "C" int onellm_gemm_timeout_flag(void) { return onellm::gemm_tc_timeout_flag(); }
