// The grouped bfloat16 matrix product of a feed-forward made of experts, on the 5th-generation tensor cores, and its
// counterpart for a handful of rows.
//
// Rows arrive sorted by expert in runs padded to whole tiles of 128 rows (csrc/moe.cu); tile i of the rows multiplies the
// matrix of expert tile_expert[i], and tiles whose entry is -1 (beyond the last run) are skipped:
//     C[128 i .. 128 i + 127, :] = A[128 i .. 128 i + 127, :] W[tile_expert[i]]^T,    W stacked [experts * n, k].
//
// * The tile kernel (prompt-sized steps) is the tile shape of csrc/gemm_tcgen05.cu with the weight tile's row taken from the
//   tile list: one persistent block per SM walks 128 x BN tiles, warp 0 (one lane) fetches operand tiles with TMA into a ring,
//   one lane of warp 1 issues tcgen05.mma (kind::f16, M 128, N BN, K 16) into two accumulators in tensor memory that alternate,
//   warps 2-5 drain a finished accumulator while the next tile's products run.  All three roles read the tile list (written by
//   the plan kernel just before) and skip the same tiles, so their counters stay in step.  Every wait is bounded; when one runs
//   out the status word says so, all roles leave their loops, tensor memory is freed and the block returns.
// * The rows kernel (steps of a few tokens) streams each used expert's matrix once: a block takes the real rows of one
//   tile (tile_rows[i] of them, eight at a time) into shared memory and its warps walk output columns, every lane reading
//   16 bytes of the matrix row per step.  Such a step is bound by the bytes of the matrices it touches, not by arithmetic.
#include "gemm_tcgen05.cuh"

namespace {
template <int BN>
struct GroupedLayout {
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int ROOM = 227 * 1024 - 1024 - 256;
    static constexpr int STAGES = ROOM / STAGE_BYTES > 6 ? 6 : ROOM / STAGE_BYTES;
    static constexpr int ACC_STRIDE = 256;  // columns between the two accumulators
    static constexpr int TMEM_COLS = 512;
    static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + 256;
};

struct GroupedParams {
    bf16* c;                 // [rows, n]
    const int* tile_expert;  // [tiles_m]
    int rows, n, k, ldc;     // n: columns per expert
    int* status;
};

template <int BN>
__device__ __forceinline__ void store_grouped_row(const GroupedParams& p, unsigned lane_addr, int r, int col0) {
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
        float v[16];
        tmem_ld16(lane_addr + c, v);
        const int col = col0 + c;
        if (r < p.rows && col < p.n) {
            bf16* dst = p.c + (size_t)r * p.ldc + col;
            if (col + 16 <= p.n && (p.ldc & 7) == 0) {
                uint4 w[2];
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(w);
#pragma unroll
                for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                reinterpret_cast<uint4*>(dst)[0] = w[0];
                reinterpret_cast<uint4*>(dst)[1] = w[1];
            } else {
                for (int j = 0; j < 16 && col + j < p.n; ++j) dst[j] = __float2bfloat16_rn(v[j]);
            }
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(THREADS) gemm_grouped_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                                                               const GroupedParams p, int tiles_m, int tiles_n) {
    using L = GroupedLayout<BN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(tiles + (size_t)L::STAGES * L::STAGE_BYTES);
    unsigned long long* empty = full + L::STAGES;
    unsigned long long* acc_full = empty + L::STAGES;  // [2]
    unsigned long long* acc_empty = acc_full + 2;      // [2]
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
    volatile int* failed = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    let_next_kernel_start();
    const int total = tiles_m * tiles_n;
    const int k_blocks = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < L::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;
    // the tile list and the rows come from the kernels before: nothing is read ahead of them
    wait_for_previous_kernels();

    if (warp == 0) {
        if (lane == 0) {  // producer
            int s = 0;
            unsigned turn = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const int tile_m = t % tiles_m, tile_n = t / tiles_m;
                const int expert = p.tile_expert[tile_m];
                if (expert < 0) continue;
                const int row0 = tile_m * BM, w_row0 = expert * p.n + tile_n * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_ready(smem_u32(&empty[s]), turn ^ 1u) && !mbar_wait(&empty[s], turn ^ 1u, failed)) { *failed = 1; ok = false; break; }
                    unsigned char* a_tile = tiles + (size_t)s * L::STAGE_BYTES;
                    mbar_expect_tx(&full[s], L::STAGE_BYTES);
                    tma_load_2d(a_tile, &map_x, &full[s], kb * BK, row0);
                    tma_load_2d(a_tile + L::A_BYTES, &map_w, &full[s], kb * BK, w_row0);
                    if (++s == L::STAGES) { s = 0; turn ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // tensor-core issuer
            const unsigned idesc = umma_idesc(BN);
            const unsigned a_low0 = desc_low(tiles), b_low0 = desc_low(tiles + L::A_BYTES), step = (unsigned)L::STAGE_BYTES >> 4;
            const unsigned full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]);
            int s = 0, i = 0;
            unsigned turn = 0, a_low = a_low0, b_low = b_low0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                if (p.tile_expert[t % tiles_m] < 0) continue;
                const int buf = i & 1;
                if (!mbar_wait(&acc_empty[buf], ((i >> 1) & 1) ^ 1, failed)) { *failed = 1; ok = false; break; }  // the epilogue has drained it
                tc_fence_after();
                const unsigned acc = tmem + buf * L::ACC_STRIDE;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_ready(full0 + 8u * (unsigned)s, turn) && !mbar_wait(&full[s], turn, failed)) { *failed = 1; ok = false; break; }
                    umma_stage(acc, a_low, b_low, idesc, kb > 0 ? 1u : 0u);
                    umma_commit_at(empty0 + 8u * (unsigned)s);  // the stage is free once these products have read it
                    a_low += step;
                    b_low += step;
                    if (++s == L::STAGES) { s = 0; turn ^= 1u; a_low = a_low0; b_low = b_low0; }
                }
                if (ok) umma_commit(&acc_full[buf]);
                ++i;
            }
        }
    } else {  // epilogue: warps 2..5 read TMEM lane quarters 2, 3, 0, 1
        const int quarter = warp & 3;
        bool ok = true;
        int i = 0;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            const int tile_m = t % tiles_m, tile_n = t / tiles_m;
            if (p.tile_expert[tile_m] < 0) continue;
            const int buf = i & 1;
            if (!mbar_wait(&acc_full[buf], (i >> 1) & 1, failed)) { *failed = 1; ok = false; break; }
            tc_fence_after();
            store_grouped_row<BN>(p, tmem + buf * L::ACC_STRIDE + ((unsigned)(quarter * 32) << 16), tile_m * BM + quarter * 32 + lane, tile_n * BN);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {  // this warp's quarter of the accumulator may be written again
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
            }
            ++i;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *failed) atomicOr(p.status, HB_STATUS_WAIT_EXPIRED | HB_STATUS_IN_GEMM_TILES);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
    }
}

template <int BN>
int launch_grouped(const CUtensorMap& map_x, const CUtensorMap& map_w, const GroupedParams& p, int tiles_m, int tiles_n, int blocks, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_grouped_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GroupedLayout<BN>::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_after_previous(gemm_grouped_kernel<BN>, dim3(blocks), THREADS, GroupedLayout<BN>::SMEM, stream, map_x, map_w, p, tiles_m, tiles_n);
}

// ---------------------------------------------------------------- a few rows per expert: the matrices stream once
constexpr int ROWS_AT_ONCE = 8, COLUMNS_PER_BLOCK = 32, ROWS_THREADS = 256;

__global__ void __launch_bounds__(ROWS_THREADS) gemm_grouped_rows_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, bf16* __restrict__ c,
                                                                         const int* __restrict__ tile_expert, const int* __restrict__ tile_rows, int pad,
                                                                         int n, int k) {
    extern __shared__ __align__(16) unsigned char rows_raw[];
    bf16* rows = reinterpret_cast<bf16*>(rows_raw);  // [ROWS_AT_ONCE, k]
    let_next_kernel_start();
    wait_for_previous_kernels();  // the tile list and the rows come from the kernels before
    const int tile = blockIdx.y;
    const int expert = tile_expert[tile];
    if (expert < 0) return;
    const int real = tile_rows[tile];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* we = w + (size_t)expert * n * k;
    const int chunks = k / 8;  // 16-byte pieces of a row
    for (int first = 0; first < real; first += ROWS_AT_ONCE) {
        const int count = min(ROWS_AT_ONCE, real - first);
        __syncthreads();
        for (int e = threadIdx.x; e < ROWS_AT_ONCE * chunks; e += ROWS_THREADS) {
            const int r = e / chunks, piece = e - r * chunks;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (r < count) value = *reinterpret_cast<const uint4*>(a + (size_t)(tile * pad + first + r) * k + piece * 8);
            *reinterpret_cast<uint4*>(rows + (size_t)r * k + piece * 8) = value;
        }
        __syncthreads();
        for (int j = warp; j < COLUMNS_PER_BLOCK; j += ROWS_THREADS / 32) {
            const int col = blockIdx.x * COLUMNS_PER_BLOCK + j;
            if (col >= n) break;
            const bf16* wrow = we + (size_t)col * k;
            float sum[ROWS_AT_ONCE];
#pragma unroll
            for (int r = 0; r < ROWS_AT_ONCE; ++r) sum[r] = 0.f;
            for (int piece = lane; piece < chunks; piece += 32) {
                const uint4 raw = *reinterpret_cast<const uint4*>(wrow + piece * 8);
                const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&raw);
                float wf[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(wp[i]); wf[2 * i] = f.x; wf[2 * i + 1] = f.y; }
#pragma unroll
                for (int r = 0; r < ROWS_AT_ONCE; ++r) {
                    const uint4 xr = *reinterpret_cast<const uint4*>(rows + (size_t)r * k + piece * 8);
                    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xr);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(xp[i]);
                        sum[r] = fmaf(f.x, wf[2 * i], sum[r]);
                        sum[r] = fmaf(f.y, wf[2 * i + 1], sum[r]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < ROWS_AT_ONCE; ++r) sum[r] = warp_sum(sum[r]);
            if (lane < count) {
                float mine = sum[0];
#pragma unroll
                for (int r = 1; r < ROWS_AT_ONCE; ++r)
                    if (lane == r) mine = sum[r];
                c[(size_t)(tile * pad + first + lane) * n + col] = __float2bfloat16_rn(mine);
            }
        }
    }
}
}  // namespace

// a [rows, k] and c [rows, n] dense bfloat16 (rows a multiple of 128), w [experts, n, k] dense bfloat16, k a multiple of 8.
HB_EXPORT int hb_moe_gemm_tiles(const void* a, const void* w, void* c, const int* tile_expert, int rows, int experts, int n, int k, int* status,
                                cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return 0;
    if (k <= 0 || rows % BM || experts <= 0 || (k % 8) || !tile_expert) return HB_BAD_ARGUMENT;
    if ((long long)experts * n > 0x7fffffffLL) return HB_UNSUPPORTED_SIZE;
    const int bn = n % 256 == 0 || n >= 1024 ? 256 : 128;
    CUtensorMap map_x, map_w;
    if (int code = make_map(&map_x, a, rows, k, k, BM)) return code;
    if (int code = make_map(&map_w, w, experts * n, k, k, bn)) return code;
    const int tiles_m = rows / BM, tiles_n = (n + bn - 1) / bn;
    if ((long long)tiles_m * tiles_n > 0x7fffffffLL) return HB_UNSUPPORTED_SIZE;
    const int blocks = min(tiles_m * tiles_n, sm_count());
    const GroupedParams p{(bf16*)c, tile_expert, rows, n, k, n, status};
    return bn == 256 ? launch_grouped<256>(map_x, map_w, p, tiles_m, tiles_n, blocks, stream)
                     : launch_grouped<128>(map_x, map_w, p, tiles_m, tiles_n, blocks, stream);
}

// The same product for steps of a few rows; tile_rows[i]: the real rows at the start of tile i.
HB_EXPORT int hb_moe_gemm_rows(const void* a, const void* w, void* c, const int* tile_expert, const int* tile_rows, int pad, int rows, int n, int k,
                               cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return 0;
    if (k <= 0 || pad <= 0 || rows % pad || (k % 8) || !tile_expert || !tile_rows) return HB_BAD_ARGUMENT;
    if ((((uintptr_t)a | (uintptr_t)w) & 15)) return HB_BAD_ARGUMENT;
    const size_t shared = (size_t)ROWS_AT_ONCE * k * sizeof(bf16);
    if (shared > 200 * 1024 || rows / pad > 65535) return HB_UNSUPPORTED_SIZE;
    static size_t configured = 48 * 1024;
    if (shared > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_grouped_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (e != cudaSuccess) return (int)e;
        configured = shared;
    }
    const dim3 grid((n + COLUMNS_PER_BLOCK - 1) / COLUMNS_PER_BLOCK, rows / pad);
    return launch_after_previous(gemm_grouped_rows_kernel, grid, dim3(ROWS_THREADS), shared, stream, (const bf16*)a, (const bf16*)w, (bf16*)c, tile_expert,
                                 tile_rows, pad, n, k);
}
