// Expert products for many tokens: the (token, expert) pairs of a step sorted by expert, then one tiled bfloat16
// matrix product over all experts at once (mma.sync m16n8k16, 32-bit accumulation).
//
//   plan     one block: counts the pairs of every expert, lays the experts' pairs out one after the other, deals
//            each expert's rows into tiles of 128 and notes, for every pair, the row it got.  Which row of its
//            expert's run a pair gets depends on the order in which threads arrive; a row's result does not depend
//            on its place, so the step's result does not either.
//   product  one block per (row tile, column tile): C[r, n] = sum_k A[row_of(r), k] * W[expert][n, k].  A rows are
//            gathered through the plan (the token of the pair) or taken as they lie (the rows the first product
//            wrote).  K and W tiles travel by cp.async through a three-stage ring into XOR-swizzled shared tiles;
//            eight warps hold 64 x 32 outputs each.  Two forms: *gated*, where W holds an expert's gate rows and then
//            its up rows and a tile takes 64 features' gate rows and the same features' up rows in alternating
//            groups of eight, so that a thread holds both halves of an output and writes
//                min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1)
//            rounded once to bfloat16; and *plain*, which writes the 32-bit sums.
#include "common.cuh"

namespace {

constexpr int kBlockRows = 128;      // pairs per tile
constexpr int kBlockCols = 128;      // rows of W per tile (gated: 64 features, gate and up)
constexpr int kBlockInner = 64;      // k per stage: one 128-byte row of bfloat16
constexpr int kStages = 3;
constexpr int kGemmThreads = 256;

__device__ __forceinline__ uint32_t shared_address(const void* pointer) { return (uint32_t)__cvta_generic_to_shared(pointer); }
__device__ __forceinline__ void copy_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void load_matrices(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// element offset of (row, 16-byte chunk) in a tile whose rows hold 64 bfloat16
__device__ __forceinline__ int tile_at(int row, int chunk) { return row * kBlockInner + ((chunk ^ (row & 7)) << 3); }

}  // namespace

// plan[0] = number of row tiles; then per tile (expert, first row, rows); see llm_moe_plan for the other outputs.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ chosen, int n_pairs, int experts,
                                                        int* __restrict__ offsets, int* __restrict__ pair_of_row,
                                                        int* __restrict__ row_of_pair, int* __restrict__ tiles, int max_tiles) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int plan_shared[];     // [experts] counts, then cursors; [experts + 1] offsets
    int* count = plan_shared;
    int* start = plan_shared + experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(count + chosen[p], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0, tile = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = total;
            offsets[e] = total;
            for (int row = 0; row < count[e] && tile < max_tiles; row += kBlockRows, ++tile) {
                tiles[1 + 3 * tile] = e;
                tiles[2 + 3 * tile] = total + row;
                tiles[3 + 3 * tile] = min(kBlockRows, count[e] - row);
            }
            total += count[e];
        }
        start[experts] = total;
        offsets[experts] = total;
        tiles[0] = tile;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;     // now the cursors
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = chosen[p];
        const int row = start[e] + atomicAdd(count + e, 1);
        pair_of_row[row] = p;
        row_of_pair[p] = row;
    }
}

template <bool GATED>
__global__ void __launch_bounds__(kGemmThreads) moe_grouped_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w,
                                                                   const int* __restrict__ tiles, const int* __restrict__ pair_of_row,
                                                                   int in_div, void* __restrict__ out, int out_cols, int inner,
                                                                   float limit, float alpha, float up_shift) {
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= tiles[0]) return;
    extern __shared__ __align__(128) unsigned char grouped_shared[];
    __nv_bfloat16* a_tiles = reinterpret_cast<__nv_bfloat16*>(grouped_shared);                   // [stages][128][64]
    __nv_bfloat16* w_tiles = a_tiles + kStages * kBlockRows * kBlockInner;                        // [stages][128][64]
    __shared__ int source_row[kBlockRows];

    const int expert = tiles[1 + 3 * blockIdx.x], first_row = tiles[2 + 3 * blockIdx.x], n_rows = tiles[3 + 3 * blockIdx.x];
    // out_cols: columns of the output (gated: features); a column tile covers 64 features (gated) or 128 columns
    const int col0 = blockIdx.y * (GATED ? kBlockCols / 2 : kBlockCols);
    const __nv_bfloat16* matrix = w + (size_t)expert * (GATED ? 2 : 1) * out_cols * inner;
    for (int r = threadIdx.x; r < kBlockRows; r += kGemmThreads)
        source_row[r] = r < n_rows ? (pair_of_row ? pair_of_row[first_row + r] / in_div : first_row + r) : -1;
    __syncthreads();

    const int chunk = threadIdx.x & 7, row0 = threadIdx.x >> 3;      // 8 chunks per row, 32 rows per pass
    auto load_stage = [&](int stage, int k0) {
        __nv_bfloat16* a_tile = a_tiles + stage * kBlockRows * kBlockInner;
        __nv_bfloat16* w_tile = w_tiles + stage * kBlockCols * kBlockInner;
#pragma unroll
        for (int pass = 0; pass < kBlockRows / 32; ++pass) {
            const int row = row0 + pass * 32;
            const int source = source_row[row];
            const __nv_bfloat16* src = a + (size_t)(source < 0 ? 0 : source) * inner + k0 + chunk * 8;
            copy_async_16(shared_address(a_tile + tile_at(row, chunk)), src, source < 0 ? 0 : 16);
        }
#pragma unroll
        for (int pass = 0; pass < kBlockCols / 32; ++pass) {
            const int row = row0 + pass * 32;
            int global_row;
            bool valid;
            if (GATED) {      // groups of eight rows alternate between gate and up rows of the same features
                const int group = row >> 3;
                const int feature = col0 + (group >> 1) * 8 + (row & 7);
                valid = feature < out_cols;
                global_row = (group & 1 ? out_cols : 0) + feature;
            } else {
                global_row = col0 + row;
                valid = global_row < out_cols;
            }
            const __nv_bfloat16* src = matrix + (size_t)(valid ? global_row : 0) * inner + k0 + chunk * 8;
            copy_async_16(shared_address(w_tile + tile_at(row, chunk)), src, valid ? 16 : 0);
        }
    };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warp_row = (warp >> 2) * 64, warp_col = (warp & 3) * 32;
    const int matrix_index = lane >> 3, matrix_row = lane & 7;
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int v = 0; v < 4; ++v) acc[i][j][v] = 0.0f;

    const int k_tiles = inner / kBlockInner;
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (s < k_tiles) load_stage(s, s * kBlockInner);
        copy_async_commit();
    }
    for (int kt = 0; kt < k_tiles; ++kt) {
        copy_async_wait<kStages - 2>();
        __syncthreads();      // stage kt has arrived for everyone, and everyone is done with stage kt - 1
        const int next = kt + kStages - 1;
        if (next < k_tiles) load_stage(next % kStages, next * kBlockInner);
        copy_async_commit();
        const __nv_bfloat16* a_tile = a_tiles + (kt % kStages) * kBlockRows * kBlockInner;
        const __nv_bfloat16* w_tile = w_tiles + (kt % kStages) * kBlockCols * kBlockInner;
#pragma unroll
        for (int ks = 0; ks < kBlockInner / 16; ++ks) {
            uint32_t a_frag[4][4], b_frag[2][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = warp_row + i * 16 + (matrix_index & 1) * 8 + matrix_row;
                load_matrices(a_frag[i], shared_address(a_tile + tile_at(row, 2 * ks + (matrix_index >> 1))));
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int row = warp_col + j * 16 + (matrix_index >> 1) * 8 + matrix_row;
                load_matrices(b_frag[j], shared_address(w_tile + tile_at(row, 2 * ks + (matrix_index & 1))));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    mma_16816(acc[i][2 * j], a_frag[i], b_frag[j][0], b_frag[j][1]);
                    mma_16816(acc[i][2 * j + 1], a_frag[i], b_frag[j][2], b_frag[j][3]);
                }
        }
    }
    copy_async_wait<0>();

    // a thread holds rows g and g + 8 of each 16-row tile and columns 2 t, 2 t + 1 of each 8-column tile
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = warp_row + i * 16 + g + 8 * half;
            if (row >= n_rows) continue;
            const size_t out_row = (size_t)(first_row + row);
            if (GATED) {
                // column tiles 2 j (gate) and 2 j + 1 (up) of this warp belong to features col0 + warp_col / 2 + 8 j ..
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + out_row * out_cols;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int feature = col0 + warp_col / 2 + j * 8 + 2 * t;
                    float y[2];
#pragma unroll
                    for (int v = 0; v < 2; ++v) {
                        const float gate = fminf(acc[i][2 * j][2 * half + v], limit);
                        const float up = fminf(fmaxf(acc[i][2 * j + 1][2 * half + v], -limit), limit);
                        y[v] = gate / (1.0f + __expf(-alpha * gate)) * (up + up_shift);
                    }
                    if (feature + 1 < out_cols) {
                        *reinterpret_cast<__nv_bfloat162*>(dst + feature) = __floats2bfloat162_rn(y[0], y[1]);
                    } else if (feature < out_cols) {
                        dst[feature] = __float2bfloat16_rn(y[0]);
                    }
                }
            } else {
                float* dst = reinterpret_cast<float*>(out) + out_row * out_cols;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int column = col0 + warp_col + j * 8 + 2 * t;
                    if (column + 1 < out_cols) {
                        *reinterpret_cast<float2*>(dst + column) = make_float2(acc[i][j][2 * half], acc[i][j][2 * half + 1]);
                    } else if (column < out_cols) {
                        dst[column] = acc[i][j][2 * half];
                    }
                }
            }
        }
    }
}

// out[t] = sum_j weight[t, j] * down[row_of_pair[t * top + j]] (+ shared[t]), 32-bit, slots in order.
template <typename T>
__global__ void moe_combine_rows_kernel(const float* __restrict__ down, const int* __restrict__ row_of_pair,
                                        const float* __restrict__ weights, const T* __restrict__ shared_out, T* __restrict__ out,
                                        int width, int top) {
    pdl_trigger();
    pdl_wait();
    const size_t token = blockIdx.x;
    for (int column = threadIdx.x * 4; column < width; column += blockDim.x * 4) {
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int j = 0; j < top; ++j) {
            const float weight = weights[token * top + j];
            const float4 value = *reinterpret_cast<const float4*>(down + (size_t)row_of_pair[token * top + j] * width + column);
            sum[0] = fmaf(weight, value.x, sum[0]);
            sum[1] = fmaf(weight, value.y, sum[1]);
            sum[2] = fmaf(weight, value.z, sum[2]);
            sum[3] = fmaf(weight, value.w, sum[3]);
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (shared_out) sum[v] += Num<T>::load(shared_out + token * width + column + v);
            Num<T>::store(out + token * width + column + v, sum[v]);
        }
    }
}

// Sorts the pairs by expert.  chosen: int32 [n_pairs]; offsets: int32 [experts + 1]; pair_of_row, row_of_pair: int32
// [n_pairs]; tiles: int32 [1 + 3 * max_tiles] with max_tiles >= ceil(n_pairs / 128) + experts.
LLM_EXPORT int llm_moe_plan(const int* chosen, int n_pairs, int experts, int* offsets, int* pair_of_row, int* row_of_pair,
                            int* tiles, int max_tiles, cudaStream_t stream) {
    if (n_pairs == 0) return LLM_OK;
    if (max_tiles < (n_pairs + kBlockRows - 1) / kBlockRows + experts) {
        llm_set_error("moe_plan: room for %d tiles, %d pairs of %d experts may need %d", max_tiles, n_pairs, experts,
                      (n_pairs + kBlockRows - 1) / kBlockRows + experts);
        return LLM_REFUSED;
    }
    const size_t shared = (size_t)(2 * experts + 1) * sizeof(int);
    if (shared > 40 * 1024) {
        llm_set_error("moe_plan: %d experts are too many", experts);
        return LLM_REFUSED;
    }
    llm_launch(moe_plan_kernel, 1, 1024, shared, stream, chosen, n_pairs, experts, offsets, pair_of_row, row_of_pair, tiles, max_tiles);
    return llm_check_launch("moe_plan");
}

LLM_EXPORT int llm_moe_grouped_supports(int out_cols, int inner, int gated) {
    return inner > 0 && inner % kBlockInner == 0 && out_cols > 0 && out_cols % 8 == 0 && (gated || out_cols % 4 == 0);
}

// One product over all tiles of the plan.  a: bfloat16 [*, inner]; w: bfloat16 [experts, (gated ? 2 : 1) * out_cols,
// inner]; pair_of_row null: row r of the plan reads row r of a, else row pair_of_row[r] / in_div; out: bfloat16
// [n_pairs, out_cols] (gated) or float32 [n_pairs, out_cols], rows in the plan's order.
LLM_EXPORT int llm_moe_grouped(const void* a, const void* w, const int* tiles, const int* pair_of_row, int in_div, void* out,
                               int out_cols, int inner, int max_tiles, int gated, float limit, float alpha, float up_shift, cudaStream_t stream) {
    if (max_tiles <= 0) return LLM_OK;
    if (!llm_moe_grouped_supports(out_cols, inner, gated) || in_div <= 0) {
        llm_set_error("moe_grouped: %d output columns over an inner size of %d are not supported (inner a multiple of %d, "
                      "columns a multiple of 8)", out_cols, inner, kBlockInner);
        return LLM_REFUSED;
    }
    const size_t shared = (size_t)kStages * (kBlockRows + kBlockCols) * kBlockInner * sizeof(__nv_bfloat16);
    const int per_tile = gated ? kBlockCols / 2 : kBlockCols;
    dim3 grid(max_tiles, (out_cols + per_tile - 1) / per_tile);
    if (grid.y > 65535) {
        llm_set_error("moe_grouped: %d output columns are too many for one launch", out_cols);
        return LLM_REFUSED;
    }
    if (gated) {
        if (int status = llm_raise_shared_limit((const void*)moe_grouped_kernel<true>, shared, "moe_grouped")) return status;
        llm_launch(moe_grouped_kernel<true>, grid, kGemmThreads, shared, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                   tiles, pair_of_row, in_div, out, out_cols, inner, limit, alpha, up_shift);
    } else {
        if (int status = llm_raise_shared_limit((const void*)moe_grouped_kernel<false>, shared, "moe_grouped")) return status;
        llm_launch(moe_grouped_kernel<false>, grid, kGemmThreads, shared, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                   tiles, pair_of_row, in_div, out, out_cols, inner, limit, alpha, up_shift);
    }
    return llm_check_launch("moe_grouped");
}

LLM_EXPORT int llm_moe_combine_rows(const float* down, const int* row_of_pair, const float* weights, const void* shared_out,
                                    void* out, int n_tokens, int width, int top, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (width % 4) {
        llm_set_error("moe_combine_rows: the width %d is no multiple of 4", width);
        return LLM_REFUSED;
    }
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(moe_combine_rows_kernel<T>, n_tokens, 256, 0, stream, down, row_of_pair, weights,
                                  (const T*)shared_out, (T*)out, width, top)));
    return llm_check_launch("moe_combine_rows");
}
