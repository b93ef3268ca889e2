// Dense part of the NN-Descent local join on the 5th-generation tensor cores.
//
// One tile covers two nodes: M = 128 rows (node A's new rows, node B's new rows, node A's old rows, node B's old
// rows, 32 each), N = 64 columns (the first 64 rows, i.e. both nodes' new rows, used as the B operand straight out
// of the A tile's shared memory), K = 1024 halves.  D = A x B^T accumulates in fp32 in tensor memory; the two
// diagonal 64 x 32 blocks are the joins' dense inner products and go to the scratch layout
// D[node][participant 0..63][new row 0..31] that the sparse half of the join reads.  Inputs are exact halves and
// accumulation is fp32, so the result has fp32-level accuracy without splitting operands.
//
// Rows are gathered from arbitrary documents, so operands cannot come from a tiled tensor map: four producer warps
// copy 16-byte pieces with cp.async straight into the 128-byte-swizzled K-major layout the MMA descriptors
// expect, three 64 KB stages (K = 256 each) in flight; one thread issues tcgen05.mma and commits each stage back
// to the producers; four epilogue warps read the accumulator with tcgen05.ld and store it.  Two accumulators
// (2 x 64 tensor-memory columns) let the epilogue of one tile overlap the MMAs of the next.  Every wait is bounded.
#include <algorithm>
#include <cstdio>

#include "apoe_common.cuh"

namespace apoe {

constexpr int kPart = 64, kNewMax = 32;
constexpr int kTcThreads = 288;          // warps 0-3 epilogue, 4-7 producers, 8 MMA issue + tensor-memory owner
constexpr int kStages = 3;
constexpr int kStageK = 256;             // halves of K per stage
constexpr int kAtomsPerStage = kStageK / 64;
constexpr int kStageBytes = 128 * kStageK * 2;   // 64 KB
constexpr int kKStages = AP_DIM / kStageK;       // 4 stages per tile
constexpr uint32_t kTmemCols = 128;
constexpr uint32_t kWaitLimit = 1u << 22;

struct TcArgs {
    uint32_t node0, nodes;
    const uint32_t *plist, *pcnt;
    const uint64_t *meta;
    const uint8_t *rec;
    float *D;
    uint32_t *err;
};

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
// K-major operand, 128-byte swizzle: 8-row groups 1024 bytes apart; descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16: D fp32 (bit 4), A and B fp16 K-major, N = 64 (bits 17-22 = N >> 3), M = 128 (bits 24-28 = M >> 4)
constexpr uint32_t kIdesc = (1u << 4) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ bool wait_or_flag(uint64_t *bar, uint32_t parity, uint32_t *err, uint32_t code) {
    for (uint32_t i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, code);
    return false;
}

__global__ void __launch_bounds__(kTcThreads, 1) join_dense_tc_kernel(const TcArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of every stage (swizzle atoms are 8 rows x 128 bytes)
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full_bar[kStages], empty_bar[kStages], tfull_bar[2], tempty_bar[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ const uint8_t *row_src[2][128];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t tiles = (a.nodes + 1) / 2;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 128); mbar_init(&empty_bar[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 4); }
        mbar_fence_init();
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    bool ok = true;

    if (warp >= 4 && warp < 8) {
        // ---------------- producers ----------------------------------------------------------------------
        const int pt = tid - 128;           // 0..127
        const int pw = pt >> 5;             // rows pw, pw + 4, ...
        uint32_t g = 0;                      // stage counter across tiles
        uint32_t signalled = 0;              // stages already handed to the MMA thread
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const uint32_t par = (tile / gridDim.x) & 1u;
            {   // which document feeds tile row `pt`
                const uint32_t blk = pt >> 5, l = pt & 31;
                const uint32_t local = tile * 2 + (blk & 1u);
                const uint8_t *src = nullptr;
                if (local < a.nodes) {
                    const uint32_t v = a.node0 + local;
                    const uint32_t n_new = a.pcnt[(size_t)v * 2], rows = a.pcnt[(size_t)v * 2 + 1];
                    const uint32_t j = blk < 2 ? l : n_new + l;
                    const bool valid = blk < 2 ? l < n_new : j < rows;
                    if (valid) src = a.rec + meta_off16(a.meta[a.plist[(size_t)v * kPart + j]]) * 16ull;
                }
                row_src[par][pt] = src;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            for (int ks = 0; ks < kKStages && ok; ++ks, ++g) {
                const uint32_t s = g % kStages;
                ok = wait_or_flag(&empty_bar[s], ((g / kStages) & 1u) ^ 1u, a.err, 10u);
                if (!ok) break;
                const uint32_t stage_base = smem_u32(smem + (size_t)s * kStageBytes);
                // chunk q = row * 32 + c: c-th 16-byte piece of the row's 512-byte K slice
#pragma unroll 4
                for (int i = 0; i < 32; ++i) {
                    const int r = pw + 4 * i;
                    const uint8_t *src = row_src[par][r];
                    const int c = lane, ka = c >> 3, cc = c & 7;
                    const uint32_t dst = stage_base + ka * (128 * 128) + r * 128 + ((cc ^ (r & 7)) << 4);
                    if (src) cp_async16(dst, src + (size_t)ks * (kStageK * 2) + c * 16);
                }
                cp_async_commit();
                if (g - signalled >= 2) {   // two younger groups may stay in flight
                    cp_async_wait<2>();
                    fence_proxy_async_smem();
                    mbar_arrive(&full_bar[signalled % kStages]);
                    ++signalled;
                }
            }
        }
        // drain
        cp_async_wait<0>();
        fence_proxy_async_smem();
        for (; signalled < g; ++signalled) mbar_arrive(&full_bar[signalled % kStages]);
    } else if (warp == 8) {
        // ---------------- MMA issue ----------------------------------------------------------------------
        uint32_t g = 0, t_local = 0;
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++t_local) {
            const uint32_t acc = t_local & 1u;
            if (lane == 0) {
                ok = wait_or_flag(&tempty_bar[acc], ((t_local >> 1) & 1u) ^ 1u, a.err, 11u);
                tc_fence_after();
                for (int ks = 0; ks < kKStages && ok; ++ks, ++g) {
                    const uint32_t s = g % kStages;
                    ok = wait_or_flag(&full_bar[s], (g / kStages) & 1u, a.err, 12u);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t stage_base = smem_u32(smem + (size_t)s * kStageBytes);
#pragma unroll
                    for (int ka = 0; ka < kAtomsPerStage; ++ka) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint64_t desc = umma_desc_sw128(stage_base + ka * (128 * 128) + kk * 32);
                            tc_mma_f16(tmem_base + acc * 64, desc, desc, kIdesc, (ks | ka | kk) != 0 ? 1u : 0u);
                        }
                    }
                    tc_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
                }
                if (ok) tc_commit(&tfull_bar[acc]);
            }
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            g = __shfl_sync(0xFFFFFFFFu, g, 0);
        }
    } else {
        // ---------------- epilogue: warp w owns tensor-memory lanes 32w .. 32w+31 -----------------------------
        uint32_t t_local = 0;
        for (uint32_t tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++t_local) {
            const uint32_t acc = t_local & 1u;
            ok = wait_or_flag(&tfull_bar[acc], (t_local >> 1) & 1u, a.err, 13u);
            if (!ok) break;
            tc_fence_after();
            uint32_t r[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * warp) << 16) + acc * 64 + (warp & 1) * 32;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                  "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                  "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
            const uint32_t local = tile * 2 + (warp & 1);
            if (local < a.nodes) {
                const uint32_t v = a.node0 + local;
                const uint32_t n_new = a.pcnt[(size_t)v * 2], rows = a.pcnt[(size_t)v * 2 + 1];
                const uint32_t j = warp < 2 ? (uint32_t)lane : n_new + lane;
                const bool valid = warp < 2 ? (uint32_t)lane < n_new : j < rows;
                if (valid) {
                    float4 *out = reinterpret_cast<float4 *>(a.D + ((size_t)local * kPart + j) * kNewMax);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        out[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                                             __uint_as_float(r[4 * q + 3]));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

int join_dense_tc_launch(ap_index *ix, uint32_t node0, uint32_t nodes, const uint32_t *plist, const uint32_t *pcnt, float *D,
                         cudaStream_t stream) {
    TcArgs a{node0, nodes, plist, pcnt, ix->meta, ix->rec_build, D, ix->d_ctl + 1};
    const size_t smem = (size_t)kStages * kStageBytes + 1024;
    // the attribute belongs to the current device's context, so it is set on every launch (builds on several GPUs in one process)
    AP_CUDA(cudaFuncSetAttribute(join_dense_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint32_t tiles = (nodes + 1) / 2;
    const uint32_t grid = std::min<uint32_t>(tiles, (uint32_t)ix->num_sms);
    if (grid == 0) return AP_OK;
    join_dense_tc_kernel<<<grid, kTcThreads, smem, stream>>>(a);
    AP_CUDA(cudaGetLastError());
    return AP_OK;
}

}  // namespace apoe

