// Dense feature transform of a GCN layer,  Z[M x 128] = H[M x 128] * W[128 x 128],
// fp32 in and out, TF32 multiply with fp32 accumulation on the sm_100a tensor
// cores (tcgen05.mma, accumulator in tensor memory), operands moved by TMA.
//
// The product is bandwidth-bound (1 KiB of HBM traffic per row against 32 KiB
// of tensor work), so the kernel is organised around keeping loads in flight:
//
//   persistent CTAs, one per SM, each taking row tiles of 128 rows round-robin;
//   warp 0 (one lane)  TMA producer: the tile's H rows arrive as four boxes of
//                      128 rows x 32 floats (128-byte swizzled) in a ring of
//                      GEMM_STAGES 16 KiB stages, freed by tcgen05.commit;
//   warp 1 (one lane)  MMA issuer: 16 tcgen05.mma (M128 N128 K8, kind::tf32) per
//                      tile into one of two 128-column TMEM accumulators;
//   warps 2-5          epilogue: tcgen05.ld the accumulator, transpose through a
//                      small shared-memory patch so that every store instruction
//                      writes whole 128-byte lines of Z.
//   W is loaded once per CTA into shared memory, transposed to K-major and
//   swizzled by hand (it is 64 KiB and read by every MMA).
//
// Every wait on an mbarrier is bounded: after GEMM_SPIN_LIMIT polls the thread
// records a code in *err_flag, raises a CTA-wide abort flag that every loop
// checks, and the kernel drains and frees its tensor memory before returning.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace agcn {

constexpr int GEMM_DIM = 128;                 // K and N of the product
constexpr int GEMM_TILE_M = 128;
constexpr int GEMM_KBLK = 32;                 // floats in one 128-byte swizzle row
constexpr int GEMM_KBLKS = GEMM_DIM / GEMM_KBLK;
constexpr int GEMM_STAGES = 6;
constexpr int GEMM_STAGE_BYTES = GEMM_TILE_M * GEMM_KBLK * 4;          // 16 KiB
constexpr int GEMM_W_BYTES = GEMM_DIM * GEMM_DIM * 4;                  // 64 KiB
constexpr int GEMM_PATCH_STRIDE = 36;                                  // floats per patch row (16-byte aligned, skewed)
constexpr int GEMM_PATCH_BYTES = 32 * GEMM_PATCH_STRIDE * 4;           // per epilogue warp
constexpr int GEMM_EPI_WARPS = 4;
constexpr int GEMM_THREADS = 32 * (2 + GEMM_EPI_WARPS);
constexpr int GEMM_TMEM_COLS = 256;                                    // two fp32 accumulators of 128 columns
constexpr int GEMM_SMEM_BYTES = 1024 /* alignment slack */ + GEMM_W_BYTES + GEMM_STAGES * GEMM_STAGE_BYTES +
                                GEMM_EPI_WARPS * GEMM_PATCH_BYTES + 256 /* barriers */;
constexpr uint32_t GEMM_SPIN_LIMIT = 1u << 22;     // polls (each backs off ~100 ns): about half a second

constexpr int GEMM_ERR_TIMEOUT_PRODUCER = 1, GEMM_ERR_TIMEOUT_MMA = 2, GEMM_ERR_TIMEOUT_EPILOGUE = 3;

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the barrier did not complete or the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t spin_limit)
{
    for (uint32_t spin = 0; spin < spin_limit; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (spin > 64) __nanosleep(100);
    }
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], one elected thread
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// the mbarrier is arrived on once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns of tensor memory -> 32 registers per thread
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float (&v)[32])
{
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B): 8-row groups are 1024 bytes
// apart (stride byte offset), the leading byte offset is unused for this layout.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address, bits 0-13
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused), bits 16-29
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset, bits 32-45
    d |= (uint64_t)1 << 46;                               // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                               // layout: 128-byte swizzle
    return d;
}

// Instruction descriptor of kind::tf32, fp32 accumulate, A and B K-major, M = 128, N = 128.
constexpr uint32_t GEMM_IDESC = (1u << 4)                 /* D format: f32 */
                              | (2u << 7)                 /* A format: tf32 */
                              | (2u << 10)                /* B format: tf32 */
                              | ((uint32_t)(GEMM_DIM >> 3) << 17)      /* N / 8 */
                              | ((uint32_t)(GEMM_TILE_M >> 4) << 24);  /* M / 16 */

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tf32_128_kernel(const __grid_constant__ CUtensorMap map_h, const float *__restrict__ w,
                     float *__restrict__ z, int64_t ldz, int64_t m_rows, int n_tiles, int *__restrict__ err_flag,
                     uint32_t spin_limit, int skip_first_load)
{
    // spin_limit: polls a wait may take (GEMM_SPIN_LIMIT in normal use).  skip_first_load: self-test
    // of the failure path only -- the producer leaves out the first load of the thread block, so the
    // MMA issuer's wait for it runs out and the kernel must leave through the abort path.
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *s_w = smem;                                           // 64 KiB, K-major, swizzled
    uint8_t *s_ring = smem + GEMM_W_BYTES;                         // GEMM_STAGES x 16 KiB
    float *s_patch = reinterpret_cast<float *>(s_ring + GEMM_STAGES * GEMM_STAGE_BYTES);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(s_patch) + GEMM_EPI_WARPS * GEMM_PATCH_BYTES);
    uint64_t *bar_full = s_bar;                                    // [GEMM_STAGES] TMA -> MMA
    uint64_t *bar_empty = s_bar + GEMM_STAGES;                     // [GEMM_STAGES] MMA -> TMA
    uint64_t *bar_acc_full = s_bar + 2 * GEMM_STAGES;              // [2] MMA -> epilogue
    uint64_t *bar_acc_empty = s_bar + 2 * GEMM_STAGES + 2;         // [2] epilogue -> MMA
    uint32_t *s_tmem_base = reinterpret_cast<uint32_t *>(s_bar + 2 * GEMM_STAGES + 4);
    volatile int *s_abort = reinterpret_cast<volatile int *>(s_tmem_base + 1);
    volatile int *s_never = s_abort + 1;       // stays 0: for waits that must not be cut short by the abort flag

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- prologue ----------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int i = 0; i < GEMM_STAGES; i++) { mbar_init(smem_u32(&bar_full[i]), 1); mbar_init(smem_u32(&bar_empty[i]), 1); }
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(&bar_acc_full[i]), 1); mbar_init(smem_u32(&bar_acc_empty[i]), GEMM_EPI_WARPS); }
        *s_abort = 0;
        *s_never = 0;
        fence_barrier_init();
    }
    // W[k][n] (row-major) -> B operand: row n holds its K values, 32 per 128-byte swizzled row
    for (int i = threadIdx.x; i < GEMM_DIM * GEMM_DIM; i += GEMM_THREADS) {
        const int k = i / GEMM_DIM, n = i % GEMM_DIM;
        const int chunk = ((k % GEMM_KBLK) >> 2) ^ (n & 7);
        const uint32_t off = (uint32_t)(k / GEMM_KBLK) * GEMM_STAGE_BYTES + (uint32_t)n * 128u + (uint32_t)chunk * 16u +
                             (uint32_t)(k & 3) * 4u;
        *reinterpret_cast<float *>(s_w + off) = w[i];
    }
    fence_proxy_async();                 // generic-proxy writes of W must be visible to the tensor core's reads
    if (warp == 1) tmem_alloc(smem_u32(s_tmem_base), GEMM_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;

    const int my_tiles = n_tiles > (int)blockIdx.x ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (warp == 0) {
        // ---- TMA producer ---------------------------------------------------------------------
        if (lane == 0) {
            uint32_t g = 0;      // K-blocks issued so far
            for (int it = 0; it < my_tiles && !*s_abort; it++) {
                const int tile = (int)blockIdx.x + it * (int)gridDim.x;
                for (int kb = 0; kb < GEMM_KBLKS; kb++, g++) {
                    const uint32_t s = g % GEMM_STAGES, ph = (g / GEMM_STAGES) & 1;
                    if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, s_abort, spin_limit)) {
                        if (!*s_abort) { atomicExch(err_flag, GEMM_ERR_TIMEOUT_PRODUCER); *s_abort = 1; }
                        break;
                    }
                    if (skip_first_load && g == 0) continue;      // self-test: this stage never fills
                    mbar_arrive_expect_tx(smem_u32(&bar_full[s]), GEMM_STAGE_BYTES);
                    tma_load_2d(smem_u32(s_ring + s * GEMM_STAGE_BYTES), &map_h, kb * GEMM_KBLK, tile * GEMM_TILE_M,
                                smem_u32(&bar_full[s]));
                }
            }
            if (*s_abort) {
                // copies already issued still land in shared memory: give each stage a bounded chance to finish
                for (uint32_t back = 0; back < GEMM_STAGES && back < g; back++) {
                    const uint32_t gg = g - 1 - back;
                    mbar_wait(smem_u32(&bar_full[gg % GEMM_STAGES]), (gg / GEMM_STAGES) & 1, s_never, spin_limit);
                }
            }
        }
    } else if (warp == 1) {
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
                    const uint32_t s = g % GEMM_STAGES, ph = (g / GEMM_STAGES) & 1;
                    if (!mbar_wait(smem_u32(&bar_full[s]), ph, s_abort, spin_limit)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(s_ring + s * GEMM_STAGE_BYTES);
                    const uint32_t b_addr = smem_u32(s_w + kb * GEMM_STAGE_BYTES);
#pragma unroll
                    for (int k8 = 0; k8 < GEMM_KBLK / 8; k8++) {
                        // 8 tf32 values = 32 bytes along K inside the 128-byte swizzle row
                        mma_tf32(d_tmem, make_kmajor_sw128_desc(a_addr + k8 * 32), make_kmajor_sw128_desc(b_addr + k8 * 32),
                                 GEMM_IDESC, (uint32_t)((kb | k8) != 0));
                    }
                    mma_commit(smem_u32(&bar_empty[s]));       // stage reusable once these MMAs have read it
                }
                if (!ok) {
                    if (!*s_abort) { atomicExch(err_flag, GEMM_ERR_TIMEOUT_MMA); *s_abort = 1; }
                    break;
                }
                mma_commit(smem_u32(&bar_acc_full[acc]));      // accumulator complete
            }
        }
    } else {
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
                // lane = row of the patch; write the row, then read the patch back 4 rows x 128 bytes at a time
#pragma unroll
                for (int j = 0; j < 8; j++)
                    *reinterpret_cast<float4 *>(patch + lane * GEMM_PATCH_STRIDE + j * 4) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int r = j * 4 + (lane >> 3);
                    const float4 o = *reinterpret_cast<const float4 *>(patch + r * GEMM_PATCH_STRIDE + (lane & 7) * 4);
                    if (row0 + r < m_rows)
                        *reinterpret_cast<float4 *>(z + (row0 + r) * ldz + c * 32 + (lane & 7) * 4) = o;
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
        }
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
