// Expert products for many tokens on tcgen05: the tiled product over pairs sorted by expert (see moe_grouped.cu for
// the plan), with the accumulator in tensor memory.
//
// One block per SM walks (row tile of 128 sorted pairs, column tile) pairs: A = 128 rows of the activations in the plan's order (the
// first product reads a gathered copy of the tokens' rows, the second the rows the first one wrote), B = 256 rows of
// the tile's expert's matrix, D[128, 256] in 256 columns of tensor memory.  Per 64-wide k step TMA brings A (16 KiB)
// and B (two boxes of 128 rows, 32 KiB) into a ring of four stages of 128-byte-swizzled tiles that runs on across tiles; one thread issues four
// 128 x 256 x 16 MMAs per step and frees the stage with a commit; four warps read the accumulator back, 32 columns at a
// time, and store.  The accumulator has two halves of 256 columns, so a tile's read-back runs beside the next tile's
// products.  Rows of a tile that belong to the next expert (a run's last tile) are computed and not stored.
//
//   gated   B = 128 gate rows and the same features' 128 up rows: a thread finds gate and up of an output in columns
//           j and 128 + j of its own row and writes  min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u) + 1)
//           rounded once to bfloat16;
//   plain   B = 256 rows; the 32-bit sums are written as they are.
//
// Waits are bounded: a wait that runs out sets error code 7 in the flag, every role leaves its loop, nothing is
// stored and the tensor memory is freed.
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace {

constexpr int kRows = 128;           // pairs per tile (UMMA M)
constexpr int kCols = 256;           // rows of W per tile (UMMA N)
constexpr int kInner = 64;           // k per stage
constexpr int kRing = 4;
constexpr uint32_t kABytes = kRows * kInner * 2, kBBytes = kCols * kInner * 2, kStageBytes = kABytes + kBBytes;
constexpr int kTcThreads = 192;      // warp 0: copies, warp 1: MMA issue and tensor memory, warps 2-5: epilogue

template <bool GATED>
__global__ void __launch_bounds__(kTcThreads) moe_grouped_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                    const __grid_constant__ CUtensorMap map_w,
                                                                    const int* __restrict__ tiles, void* __restrict__ out, int out_cols,
                                                                    int col_tiles, int inner, float limit, float alpha,
                                                                    float up_shift, int* __restrict__ error_flag) {
    pdl_trigger();
    pdl_wait();
    const int total = tiles[0] * col_tiles;      // (row tile, column tile) pairs; block b takes b, b + gridDim.x, ...
    if ((int)blockIdx.x >= total) return;
    extern __shared__ unsigned char tc_shared_raw[];
    __shared__ __align__(8) uint64_t full[kRing], empty[kRing], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
    const uint32_t ring = (tma::smem_u32(tc_shared_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = (inner + kInner - 1) / kInner;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kRing; ++s) {
            tma::mbar_init(tma::smem_u32(&full[s]), 1);
            tma::mbar_init(tma::smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            tma::mbar_init(tma::smem_u32(&acc_full[b]), 1);
            tma::mbar_init(tma::smem_u32(&acc_empty[b]), 4);      // one arrival per epilogue warp
        }
        tma::mbar_fence_init();
        failed = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tma::smem_u32(&tmem_slot)), "r"(2 * kCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc5::fence_before();
    __syncthreads();
    tc5::fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            int step = 0;                                  // k steps issued so far, over all of this block's tiles
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const int row_tile = t / col_tiles, col_tile = t % col_tiles;
                const int expert = tiles[1 + 3 * row_tile], first_row = tiles[2 + 3 * row_tile];
                // rows of the [experts * rows per expert, inner] weight matrix where this tile's B begins
                const int w_row0 = expert * (GATED ? 2 : 1) * out_cols + col_tile * (GATED ? kCols / 2 : kCols);
                const int w_row1 = GATED ? w_row0 + out_cols : w_row0 + kCols / 2;
                for (int kt = 0; kt < k_tiles && ok; ++kt, ++step) {
                    const int s = step % kRing;
                    if (step >= kRing) ok = tma::mbar_wait(tma::smem_u32(&empty[s]), ((step / kRing) - 1) & 1);
                    if (!ok) break;
                    const uint32_t stage = ring + s * kStageBytes, bar = tma::smem_u32(&full[s]);
                    tma::mbar_expect_tx(bar, kStageBytes);
                    tma::load_2d(stage, &map_a, bar, kt * kInner, first_row);
                    tma::load_2d(stage + kABytes, &map_w, bar, kt * kInner, w_row0);
                    tma::load_2d(stage + kABytes + kBBytes / 2, &map_w, bar, kt * kInner, w_row1);
                }
            }
            if (!ok) failed = 1;
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = tc5::instruction(kRows, kCols, false);
            bool ok = true;
            int step = 0, turn = 0;                        // turn: this block's tiles so far
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++turn) {
                const int b = turn & 1;
                if (turn >= 2) ok = tma::mbar_wait(tma::smem_u32(&acc_empty[b]), ((turn >> 1) - 1) & 1);
                if (!ok) break;
                tc5::fence_after();
                for (int kt = 0; kt < k_tiles && ok; ++kt, ++step) {
                    const int s = step % kRing;
                    ok = tma::mbar_wait(tma::smem_u32(&full[s]), (step / kRing) & 1);
                    if (!ok) break;
                    tc5::fence_after();
                    const uint32_t stage = ring + s * kStageBytes;
#pragma unroll
                    for (int ks = 0; ks < kInner / 16; ++ks)
                        tc5::mma_ss(tmem + b * kCols, tc5::desc_k_major(stage + ks * 32, 1024u),
                                    tc5::desc_k_major(stage + kABytes + ks * 32, 1024u), idesc, (kt > 0 || ks > 0) ? 1u : 0u);
                    tc5::mma_commit(tma::smem_u32(&empty[s]));
                }
                if (ok) tc5::mma_commit(tma::smem_u32(&acc_full[b]));      // arrives when the tile's last MMA is complete
            }
            if (!ok) failed = 1;
        }
    } else {
        const int quarter = warp & 3;                    // the tensor-memory lanes this warp may read
        const int row = quarter * 32 + lane;
        bool ok = true;
        int turn = 0;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++turn) {
            const int b = turn & 1;
            const int row_tile = t / col_tiles, col_tile = t % col_tiles;
            const int first_row = tiles[2 + 3 * row_tile], n_rows = tiles[3 + 3 * row_tile];
            const int col0 = col_tile * (GATED ? kCols / 2 : kCols);
            ok = tma::mbar_wait(tma::smem_u32(&acc_full[b]), (turn >> 1) & 1);
            tc5::fence_after();
            if (!ok) {
                failed = 1;
                break;
            }
            const uint32_t address = tmem + b * kCols + ((uint32_t)(quarter * 32) << 16);
            const bool store = row < n_rows;
            const size_t out_row = (size_t)(first_row + row);
            if (GATED) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + out_row * out_cols;
#pragma unroll 1
                for (int j = 0; j < kCols / 2; j += 32) {
                    uint32_t gate[32], up[32];
                    tc5::tmem_load_32(address + j, gate);
                    tc5::tmem_load_32(address + kCols / 2 + j, up);
                    if (!store) continue;
#pragma unroll
                    for (int v = 0; v < 32; v += 8) {
                        const int feature = col0 + j + v;
                        if (feature + 8 > out_cols) break;      // out_cols is a multiple of 8: vectors never straddle the edge
                        uint32_t packed[4];
#pragma unroll
                        for (int e = 0; e < 8; e += 2) {
                            float y[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const float g = fminf(__uint_as_float(gate[v + e + h]), limit);
                                const float u = fminf(fmaxf(__uint_as_float(up[v + e + h]), -limit), limit);
                                y[h] = g / (1.0f + __expf(-alpha * g)) * (u + up_shift);
                            }
                            packed[e / 2] = tc5::pack2(y[0], y[1]);
                        }
                        *reinterpret_cast<uint4*>(dst + feature) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    }
                }
            } else {
                float* dst = reinterpret_cast<float*>(out) + out_row * out_cols;
#pragma unroll 1
                for (int j = 0; j < kCols; j += 32) {
                    uint32_t sums[32];
                    tc5::tmem_load_32(address + j, sums);
                    if (!store) continue;
#pragma unroll
                    for (int v = 0; v < 32; v += 4) {
                        const int column = col0 + j + v;
                        if (column + 4 > out_cols) break;       // out_cols is a multiple of 4
                        *reinterpret_cast<float4*>(dst + column) = make_float4(__uint_as_float(sums[v]), __uint_as_float(sums[v + 1]),
                                                                                __uint_as_float(sums[v + 2]), __uint_as_float(sums[v + 3]));
                    }
                }
            }
            // this half of the tensor memory may be overwritten by the tile after the next
            tc5::fence_before();
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(tma::smem_u32(&acc_empty[b]));
        }
    }
    tc5::fence_before();
    __syncthreads();
    tc5::fence_after();
    if (failed && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 7);
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * kCols));
}

// out[r] = x[pair_of_row[r] / in_div]: the tokens' rows in the plan's order, for a product that reads its rows by TMA.
// With `pair_scale` the row of pair p is multiplied by pair_scale[p] on the way (32-bit product, one rounding): a routing
// weight that acts on what goes into an expert.
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ pair_of_row, int in_div,
                                       __nv_bfloat16* __restrict__ out, int width, const float* __restrict__ pair_scale) {
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;
    const int pair = pair_of_row[row];
    const __nv_bfloat16* from = x + (size_t)(pair / in_div) * width;
    if (pair_scale) {
        const float scale = pair_scale[pair];
        for (int i = threadIdx.x; i < width / 8; i += blockDim.x) {
            float values[8];
            load8<__nv_bfloat16>(from + i * 8, values);
#pragma unroll
            for (int j = 0; j < 8; ++j) values[j] *= scale;
            store8<__nv_bfloat16>(out + row * width + i * 8, values);
        }
        return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(from);
    uint4* dst = reinterpret_cast<uint4*>(out + row * width);
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src[i];
}

}  // namespace

LLM_EXPORT int llm_moe_grouped_tc_supports(int out_cols, int inner, int gated) {
    return inner >= 64 && inner % 8 == 0 && out_cols > 0 && out_cols % 8 == 0;
}

LLM_EXPORT int llm_moe_gather_rows(const void* x, const int* pair_of_row, int in_div, void* out, int n_rows, int width,
                                   const float* pair_scale, cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    if (width % 8 || !aligned16(x) || !aligned16(out) || in_div <= 0) {
        llm_set_error("moe_gather_rows: rows of %d elements must be a multiple of 8 and 16-byte aligned", width);
        return LLM_REFUSED;
    }
    llm_launch(moe_gather_rows_kernel, n_rows, 128, 0, stream, (const __nv_bfloat16*)x, pair_of_row, in_div, (__nv_bfloat16*)out, width,
               pair_scale);
    return llm_check_launch("moe_gather_rows");
}

// a: bfloat16 [n_rows, inner] in the plan's order; w: bfloat16 [experts, (gated ? 2 : 1) * out_cols, inner]; out: bfloat16
// [n_rows, out_cols] (gated) or float32 [n_rows, out_cols].
LLM_EXPORT int llm_moe_grouped_tc(const void* a, int n_rows, const void* w, int experts, const int* tiles, void* out, int out_cols,
                                  int inner, int max_tiles, int gated, float limit, float alpha, float up_shift, int* error_flag,
                                  cudaStream_t stream) {
    if (max_tiles <= 0 || n_rows <= 0) return LLM_OK;
    if (!llm_moe_grouped_tc_supports(out_cols, inner, gated) || !aligned16(a) || !aligned16(w) || !aligned16(out)) {
        llm_set_error("moe_grouped_tc: %d output columns over an inner size of %d are not supported (both multiples of 8, "
                      "16-byte aligned operands)", out_cols, inner);
        return LLM_REFUSED;
    }
    CUtensorMap map_a, map_w;
    const uint64_t w_rows = (uint64_t)experts * (gated ? 2 : 1) * out_cols;
    if (!tma::make_map_bf16(&map_a, a, (uint64_t)n_rows, (uint64_t)inner, kRows) ||
        !tma::make_map_bf16(&map_w, w, w_rows, (uint64_t)inner, kCols / 2)) {
        llm_set_error("moe_grouped_tc: the tensor maps could not be made");
        return LLM_REFUSED;
    }
    const size_t shared = (size_t)kRing * kStageBytes + 1024;
    const int per_tile = gated ? kCols / 2 : kCols;
    const int col_tiles = (out_cols + per_tile - 1) / per_tile;
    // one block per SM (the ring fills its shared memory); each walks the tiles b, b + blocks, ... of the plan
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    long long most = (long long)max_tiles * col_tiles;
    const int blocks = (int)(most < sms ? most : sms);
    if (gated) {
        if (int status = llm_raise_shared_limit((const void*)moe_grouped_tc_kernel<true>, shared, "moe_grouped_tc")) return status;
        llm_launch(moe_grouped_tc_kernel<true>, blocks, kTcThreads, shared, stream, map_a, map_w, tiles, out, out_cols, col_tiles, inner,
                   limit, alpha, up_shift, error_flag);
    } else {
        if (int status = llm_raise_shared_limit((const void*)moe_grouped_tc_kernel<false>, shared, "moe_grouped_tc")) return status;
        llm_launch(moe_grouped_tc_kernel<false>, blocks, kTcThreads, shared, stream, map_a, map_w, tiles, out, out_cols, col_tiles, inner,
                   limit, alpha, up_shift, error_flag);
    }
    return llm_check_launch("moe_grouped_tc");
}
