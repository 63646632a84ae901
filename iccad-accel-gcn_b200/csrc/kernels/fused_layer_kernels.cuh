// One GCN layer boundary in one kernel:  Z2[r] = relu(A[r, :] * Z1) * W  for the leading rows of a
// degree-ordered block, all of at most FUSED_MAX_DEG nonzeros.  The activations relu(A * Z1) never
// reach global memory: producer warps gather them straight into the shared-memory operand tiles of
// the tensor-core product (K-major, 128-byte swizzle -- the layout TMA writes in the plain GEMM),
// and the MMA issuer, the tensor-memory accumulators and the epilogue are those of
// gemm_tf32_128_kernel.
//
//   persistent CTAs, one per SM, each taking tiles of 128 rows round-robin;
//   warps 0, 6-31      producers: a warp owns every 27th row of the tile; it first loads the row
//                      pointers, column ids and values of all its rows (a lane holds one nonzero
//                      of each row; they are broadcast by shuffle), then gathers FUSED_ROWS rows at
//                      a time, a lane owning 4 of the 128 columns, 8 loads of 16 bytes per lane;
//   warp 1 (one lane)  MMA issuer;   warps 2-5  epilogue.
//   The operand ring holds two tiles of four K-blocks; a tile's four stage barriers are arrived on
//   by every producer warp once its rows of the tile are written and fenced for the async proxy.
// Every wait is bounded, as in the GEMM.
//
// Measured on B200 (two-layer forward, N = 5e6): correct, and slower than SpMM + GEMM -- 24.9 ms per
// forward against 14.3 ms; the dense transform it saves is 6 % of the forward.  It is therefore off
// by default (AGCN_GCN_FUSED=1 turns it on in agcn_gcn2_forward_*) and kept as the measured variant.
#pragma once
#include "gemm_tf32_kernels.cuh"
#include "ptx.cuh"

namespace agcn {

constexpr int FUSED_STAGES = 2 * GEMM_KBLKS;          // two operand tiles
constexpr int FUSED_PROD_WARPS = 27;
constexpr int FUSED_WARPS = 2 + GEMM_EPI_WARPS + FUSED_PROD_WARPS - 1;   // warp 0 is a producer too: 32 warps
constexpr int FUSED_THREADS = 32 * FUSED_WARPS;
constexpr int FUSED_ROWS = 2;                         // rows a producer warp gathers at a time
constexpr int FUSED_WARP_ROWS = (GEMM_TILE_M + FUSED_PROD_WARPS - 1) / FUSED_PROD_WARPS;   // rows of a tile per producer warp
constexpr int FUSED_MAX_DEG = 32;                     // nonzeros of a row live in one register per lane
constexpr int FUSED_ERR_BAD_COLUMN = 4;               // status code beside the GEMM_ERR_TIMEOUT_* ones
constexpr int FUSED_SMEM_BYTES = 1024 /* alignment slack */ + GEMM_W_BYTES + FUSED_STAGES * GEMM_STAGE_BYTES +
                                 GEMM_EPI_WARPS * GEMM_PATCH_BYTES + 256 /* barriers */;

__global__ void __launch_bounds__(FUSED_THREADS, 1)
gcn_fused_layer_kernel(const int *__restrict__ indptr, const int *__restrict__ idx, const float *__restrict__ val,
                       const float *__restrict__ z_in, const float *__restrict__ w, float *__restrict__ z_out,
                       int64_t m_rows, int64_t n_cols, int n_tiles, int *__restrict__ err_flag, uint32_t spin_limit)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *s_w = smem;                                           // 64 KiB, K-major, swizzled
    uint8_t *s_ring = smem + GEMM_W_BYTES;                         // FUSED_STAGES x 16 KiB
    float *s_patch = reinterpret_cast<float *>(s_ring + FUSED_STAGES * GEMM_STAGE_BYTES);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(s_patch) + GEMM_EPI_WARPS * GEMM_PATCH_BYTES);
    uint64_t *bar_full = s_bar;                                    // [FUSED_STAGES] producers -> MMA
    uint64_t *bar_empty = s_bar + FUSED_STAGES;                    // [FUSED_STAGES] MMA -> producers
    uint64_t *bar_acc_full = s_bar + 2 * FUSED_STAGES;             // [2] MMA -> epilogue
    uint64_t *bar_acc_empty = s_bar + 2 * FUSED_STAGES + 2;        // [2] epilogue -> MMA
    uint32_t *s_tmem_base = reinterpret_cast<uint32_t *>(s_bar + 2 * FUSED_STAGES + 4);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem_base + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- prologue ----------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int i = 0; i < FUSED_STAGES; i++) { mbar_init(smem_u32(&bar_full[i]), FUSED_PROD_WARPS); mbar_init(smem_u32(&bar_empty[i]), 1); }
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&bar_acc_full[i]), 1); mbar_init(smem_u32(&bar_acc_empty[i]), GEMM_EPI_WARPS); }
        *s_abort = 0;
        fence_barrier_init();
    }
    // W[k][n] (row-major) -> B operand: row n holds its K values, 32 per 128-byte swizzled row
    for (int i = threadIdx.x; i < GEMM_DIM * GEMM_DIM; i += FUSED_THREADS) {
        const int k = i / GEMM_DIM, n = i % GEMM_DIM;
        const int chunk = ((k % GEMM_KBLK) >> 2) ^ (n & 7);
        const uint32_t off = (uint32_t)(k / GEMM_KBLK) * GEMM_STAGE_BYTES + (uint32_t)n * 128u + (uint32_t)chunk * 16u +
                             (uint32_t)(k & 3) * 4u;
        *reinterpret_cast<float *>(s_w + off) = w[i];
    }
    fence_proxy_async();
    if (warp == 1) tmem_alloc(smem_u32(s_tmem_base), GEMM_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;

    const int my_tiles = n_tiles > (int)blockIdx.x ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (warp == 1) {
        // ---- MMA issuer -----------------------------------------------------------------------
        if (lane == 0) {
            uint32_t g = 0;
            for (int it = 0; it < my_tiles && !*s_abort; it++) {
                const uint32_t acc = it & 1, acc_ph = (it >> 1) & 1;
                if (!mbar_wait(smem_u32(&bar_acc_empty[acc]), acc_ph ^ 1, s_abort, spin_limit)) {
                    if (!*s_abort) { atomicExch(err_flag, GEMM_ERR_TIMEOUT_MMA); *s_abort = 1; }
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * GEMM_DIM;
                bool ok = true;
                for (int kb = 0; kb < GEMM_KBLKS; kb++, g++) {
                    const uint32_t s = g % FUSED_STAGES, ph = (g / FUSED_STAGES) & 1;
                    if (!mbar_wait(smem_u32(&bar_full[s]), ph, s_abort, spin_limit)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(s_ring + s * GEMM_STAGE_BYTES);
                    const uint32_t b_addr = smem_u32(s_w + kb * GEMM_STAGE_BYTES);
#pragma unroll
                    for (int k8 = 0; k8 < GEMM_KBLK / 8; k8++)
                        mma_tf32(d_tmem, make_kmajor_sw128_desc(a_addr + k8 * 32), make_kmajor_sw128_desc(b_addr + k8 * 32),
                                 GEMM_IDESC, (uint32_t)((kb | k8) != 0));
                    mma_commit(smem_u32(&bar_empty[s]));       // stage reusable once these MMAs have read it
                }
                if (!ok) {
                    if (!*s_abort) { atomicExch(err_flag, GEMM_ERR_TIMEOUT_MMA); *s_abort = 1; }
                    break;
                }
                mma_commit(smem_u32(&bar_acc_full[acc]));      // accumulator complete
            }
        }
    } else if (warp >= 2 && warp < 2 + GEMM_EPI_WARPS) {
        // ---- epilogue warps -------------------------------------------------------------------
        const int q = warp & 3;                                // TMEM lane quarter this warp may read
        float *patch = s_patch + (warp - 2) * (GEMM_PATCH_BYTES / 4);
        for (int it = 0; it < my_tiles && !*s_abort; it++) {
            const int tile = (int)blockIdx.x + it * (int)gridDim.x;
            const uint32_t acc = it & 1, acc_ph = (it >> 1) & 1;
            if (!mbar_wait(smem_u32(&bar_acc_full[acc]), acc_ph, s_abort, spin_limit)) {
                if (!*s_abort) { atomicExch(err_flag, GEMM_ERR_TIMEOUT_EPILOGUE); *s_abort = 1; }
                break;
            }
            tc_fence_after();
            const int64_t row0 = (int64_t)tile * GEMM_TILE_M + q * 32;
#pragma unroll 1
            for (int c = 0; c < GEMM_DIM / 32; c++) {
                float v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * GEMM_DIM + c * 32, v);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    *reinterpret_cast<float4 *>(patch + lane * GEMM_PATCH_STRIDE + j * 4) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int r = j * 4 + (lane >> 3);
                    const float4 o = *reinterpret_cast<const float4 *>(patch + r * GEMM_PATCH_STRIDE + (lane & 7) * 4);
                    if (row0 + r < m_rows)
                        *reinterpret_cast<float4 *>(z_out + (row0 + r) * GEMM_DIM + c * 32 + (lane & 7) * 4) = o;
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
        }
    } else {
        // ---- producers: relu(A * Z1) rows, written as the A operand of the product -----------------
        const int p = warp == 0 ? 0 : warp - (1 + GEMM_EPI_WARPS);       // 0 .. FUSED_PROD_WARPS - 1
        const L2Policies pol = make_l2_policies();
        bool bad_column = false;
        for (int it = 0; it < my_tiles; it++) {                 // the warp leaves the loop as one (shuffles below)
            const int tile = (int)blockIdx.x + it * (int)gridDim.x;
            const int buf = it & 1;
            const uint32_t ph = (it >> 1) & 1;
            // the MMAs that read this buffer two tiles ago must have completed
            int ok = 1;
            if (lane == 0) {
                ok = *s_abort ? 0 : 1;
                for (int kb = 0; kb < GEMM_KBLKS && ok; kb++)
                    ok = mbar_wait(smem_u32(&bar_empty[buf * GEMM_KBLKS + kb]), ph ^ 1, s_abort, spin_limit) ? 1 : 0;
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0 && !*s_abort) { atomicExch(err_flag, GEMM_ERR_TIMEOUT_PRODUCER); *s_abort = 1; }
                break;
            }
            uint8_t *tile_base = s_ring + buf * GEMM_KBLKS * GEMM_STAGE_BYTES;
            // this warp's rows of the tile: p, p + 27, ...  First every row pointer, then every row's column
            // ids and values (a lane holds one nonzero of each row), so that the dependent loads of all
            // rows travel together; then the gathers, FUSED_ROWS rows at a time.
            int cnt[FUSED_WARP_ROWS], pc[FUSED_WARP_ROWS], first[FUSED_WARP_ROWS];
            float pv[FUSED_WARP_ROWS];
#pragma unroll
            for (int k = 0; k < FUSED_WARP_ROWS; k++) {
                const int m = p + k * FUSED_PROD_WARPS;
                const int64_t r = (int64_t)tile * GEMM_TILE_M + m;
                int a = 0, b = 0;
                if (m < GEMM_TILE_M && r < m_rows) { a = indptr[r]; b = indptr[r + 1]; }
                first[k] = a;
                cnt[k] = b - a < FUSED_MAX_DEG ? b - a : FUSED_MAX_DEG;      // the host launches rows of <= 32 nonzeros only
            }
#pragma unroll
            for (int k = 0; k < FUSED_WARP_ROWS; k++) {
                pc[k] = lane < cnt[k] ? idx[first[k] + lane] : 0;
                pv[k] = lane < cnt[k] ? val[first[k] + lane] : 0.f;
            }
#pragma unroll
            for (int k0 = 0; k0 < FUSED_WARP_ROWS; k0 += FUSED_ROWS) {
                int max_cnt = 0;
#pragma unroll
                for (int q = 0; q < FUSED_ROWS; q++)
                    if (k0 + q < FUSED_WARP_ROWS) max_cnt = max_cnt > cnt[k0 + q] ? max_cnt : cnt[k0 + q];
                float4 acc[FUSED_ROWS];
#pragma unroll
                for (int q = 0; q < FUSED_ROWS; q++) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int i = 0; i < max_cnt; i += 4) {
                    // no branch around a load: a slot past the end of its row reads row 0 and is then zeroed
                    float4 v[FUSED_ROWS][4];
#pragma unroll
                    for (int q = 0; q < FUSED_ROWS; q++)
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            if (k0 + q >= FUSED_WARP_ROWS) continue;                             // compile-time
                            int col = __shfl_sync(0xffffffffu, pc[k0 + q], (i + u) & 31);       // 0 from the lanes past the row's end
                            const bool outside = (uint64_t)(int64_t)col >= (uint64_t)n_cols;
                            bad_column = bad_column || outside;
                            col = outside ? 0 : col;
                            v[q][u] = ld_x4(z_in + (int64_t)col * GEMM_DIM + 4 * lane, pol.keep);
                        }
#pragma unroll
                    for (int q = 0; q < FUSED_ROWS; q++)
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            if (k0 + q >= FUSED_WARP_ROWS) continue;
                            const bool live = i + u < cnt[k0 + q];
                            const float a = __shfl_sync(0xffffffffu, pv[k0 + q], (i + u) & 31);       // 0 past the row's end
                            const float4 x = v[q][u];
                            acc[q].x = fmaf(a, live ? x.x : 0.f, acc[q].x); acc[q].y = fmaf(a, live ? x.y : 0.f, acc[q].y);
                            acc[q].z = fmaf(a, live ? x.z : 0.f, acc[q].z); acc[q].w = fmaf(a, live ? x.w : 0.f, acc[q].w);
                        }
                }
#pragma unroll
                for (int q = 0; q < FUSED_ROWS; q++) {
                    const int m = p + (k0 + q) * FUSED_PROD_WARPS;
                    if (k0 + q < FUSED_WARP_ROWS && m < GEMM_TILE_M) {
                        const float4 h = make_float4(fmaxf(acc[q].x, 0.f), fmaxf(acc[q].y, 0.f), fmaxf(acc[q].z, 0.f), fmaxf(acc[q].w, 0.f));
                        // columns 4*lane .. 4*lane+3: K-block lane / 8, 16-byte chunk lane % 8, swizzled by the row
                        uint8_t *dst = tile_base + (lane >> 3) * GEMM_STAGE_BYTES + m * 128 + (((lane & 7) ^ (m & 7)) << 4);
                        *reinterpret_cast<float4 *>(dst) = h;
                    }
                }
            }
            fence_proxy_async();             // these generic-proxy writes are read by the tensor core
            __syncwarp();
            if (lane == 0)
                for (int kb = 0; kb < GEMM_KBLKS; kb++) mbar_arrive(smem_u32(&bar_full[buf * GEMM_KBLKS + kb]));
        }
        if (bad_column && lane == 0) atomicExch(err_flag, FUSED_ERR_BAD_COLUMN);   // that nonzero was read from row 0 instead
    }

    // ---- teardown: everyone is done (or gave up); free the tensor memory ------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, GEMM_TMEM_COLS);
    }
}

}  // namespace agcn
