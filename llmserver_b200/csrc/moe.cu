// A routed feed-forward: router, expert products taken through an index, and the weighted sum.
//
//   route      z = W_r x (32-bit), s = sigmoid(z); the `top` experts with the largest s + correction are chosen
//              (ties: the lower index), each with the weight s * scale (the correction only chooses; nothing is
//              renormalised).  One block per token.  `select` is the same choice from logits that a matrix product
//              has already made (one warp per token).
//   indexed    out[p] = W[index[p]] in[p / in_div]: every (token, chosen expert) pair p multiplies its own expert's
//   linear     matrix.  One warp per output element, its sum taken over k in an order that depends on the inner size
//              alone, so a pair's result does not depend on what else the step holds.  As a gated form the matrix
//              holds gate rows then up rows and the output is the expert's activation
//                  g = min(gate, limit), u = clamp(up, -limit, limit), y = g * sigmoid(alpha * g) * (u + up_shift)
//              computed in 32-bit and rounded once (an infinite limit, alpha 1 and up_shift 0 give silu(gate) * up).
//              With `in_scale` pair p's input row is multiplied by in_scale[p] as it is read (32-bit): a routing
//              weight that acts on what goes into an expert.  Read-once for steps of few tokens; prompts take the tiled
//              kernels of moe_grouped.cu.
//   combine    out[t] = sum_j weight[t, j] * down[t * top + j] (+ shared[t]) in 32-bit, slots in order.
#include "common.cuh"

#define MOE_MAX_TOP 32

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ x, const float* __restrict__ router, const float* __restrict__ correction,
                                 int* __restrict__ chosen, float* __restrict__ weights, int* __restrict__ counts,
                                 int width, int experts, int top, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float route_shared[];      // [width] the token's row, [experts] scores, [experts] choice scores
    float* row = route_shared;
    float* score = route_shared + width;
    float* choice = score + experts;
    const int token = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* src = x + (size_t)token * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = Num<T>::load(src + i);
    __syncthreads();
    for (int e = warp; e < experts; e += warps) {
        const float* w = router + (size_t)e * width;
        float sum = 0.0f;
        for (int i = lane; i < width; i += 32) sum = fmaf(row[i], w[i], sum);
        sum = warp_sum(sum);
        if (lane == 0) {
            const float s = 1.0f / (1.0f + expf(-sum));
            score[e] = s;
            choice[e] = s + (correction ? correction[e] : 0.0f);
        }
    }
    __syncthreads();
    if (warp != 0) return;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int best_index = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float c = choice[e];
            if (c > best) {      // within a lane indices ascend, so the first of equals stays
                best = c;
                best_index = e;
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
            if (other > best || (other == best && other_index < best_index)) {
                best = other;
                best_index = other_index;
            }
        }
        if (best_index == 0x7fffffff) best_index = 0;      // every score was NaN or -inf: never expected
        if (lane == 0) {
            chosen[(size_t)token * top + j] = best_index;
            weights[(size_t)token * top + j] = score[best_index] * scale;
            if (counts) atomicAdd(counts + best_index, 1);
            choice[best_index] = -INFINITY;
        }
        __syncwarp();
    }
}

// The choice alone, from router logits that a matrix product has made: z float32 [N, experts].  One warp per token.
__global__ void moe_select_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int* __restrict__ chosen,
                                  float* __restrict__ weights, int n_tokens, int experts, int top, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float select_shared[];      // per warp: [experts] scores, [experts] choice scores
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int token = blockIdx.x * warps + warp;
    if (token >= n_tokens) return;
    float* score = select_shared + (size_t)warp * 2 * experts;
    float* choice = score + experts;
    for (int e = lane; e < experts; e += 32) {
        const float s = 1.0f / (1.0f + expf(-logits[(size_t)token * experts + e]));
        score[e] = s;
        choice[e] = s + (correction ? correction[e] : 0.0f);
    }
    __syncwarp();
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int best_index = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float c = choice[e];
            if (c > best) {
                best = c;
                best_index = e;
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
            if (other > best || (other == best && other_index < best_index)) {
                best = other;
                best_index = other_index;
            }
        }
        if (best_index == 0x7fffffff) best_index = 0;
        if (lane == 0) {
            chosen[(size_t)token * top + j] = best_index;
            weights[(size_t)token * top + j] = score[best_index] * scale;
            choice[best_index] = -INFINITY;
        }
        __syncwarp();
    }
}

__device__ __forceinline__ float gated_activation(float gate, float up, float limit, float alpha, float up_shift = 1.0f) {
    const float g = fminf(gate, limit);
    const float u = fminf(fmaxf(up, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + up_shift);
}

// One warp per (pair, output element).  `rows` output elements per pair; the gated form reads row r and row rows + r.
template <typename T, typename O, bool GATED>
__global__ void indexed_linear_kernel(const T* __restrict__ in, const T* __restrict__ weight, const int* __restrict__ index,
                                      O* __restrict__ out, int rows, int inner, int in_div, float limit, float alpha, int index_mod,
                                      const float* __restrict__ in_scale, float up_shift) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float in_row[];       // [inner]
    const int pair = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* src = in + (size_t)(pair / in_div) * inner;
    const float row_scale = in_scale ? in_scale[pair] : 1.0f;
    for (int i = threadIdx.x; i < inner; i += blockDim.x) in_row[i] = Num<T>::load(src + i) * row_scale;
    __syncthreads();
    const int expert = index ? index[pair] : (index_mod > 0 ? pair % index_mod : 0);     // no index: pair p uses matrix p mod index_mod
    const T* matrix = weight + (size_t)expert * (GATED ? 2 : 1) * rows * inner;
    // four consecutive output elements per warp, worked on together so that their loads are in flight at the same time;
    // each element's sum runs over k in an order that depends on the inner size alone
    const int r0 = (blockIdx.y * warps + warp) * 4;
    if (r0 >= rows) return;
    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sum_up[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (inner % 8 == 0 && aligned16(weight)) {      // 16- or 32-byte runs per lane
        for (int i = lane * 8; i < inner; i += 256) {
            float values[4][8], up_values[GATED ? 4 : 1][8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int r = min(r0 + q, rows - 1);      // a warp at the edge reads the last row again and drops it below
                load8<T>(matrix + (size_t)r * inner + i, values[q]);
                if (GATED) load8<T>(matrix + ((size_t)rows + r) * inner + i, up_values[q]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float x = in_row[i + j];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    sum[q] = fmaf(x, values[q][j], sum[q]);
                    if (GATED) sum_up[q] = fmaf(x, up_values[q][j], sum_up[q]);
                }
            }
        }
    } else {
        for (int i = lane; i < inner; i += 32) {
            const float x = in_row[i];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int r = min(r0 + q, rows - 1);
                sum[q] = fmaf(x, Num<T>::load(matrix + (size_t)r * inner + i), sum[q]);
                if (GATED) sum_up[q] = fmaf(x, Num<T>::load(matrix + ((size_t)rows + r) * inner + i), sum_up[q]);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float total = warp_sum(sum[q]);
        const float total_up = GATED ? warp_sum(sum_up[q]) : 0.0f;
        if (lane == 0 && r0 + q < rows) {
            const float value = GATED ? gated_activation(total, total_up, limit, alpha, up_shift) : total;
            Num<O>::store(out + (size_t)pair * rows + r0 + q, value);
        }
    }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ down, const float* __restrict__ weights, const T* __restrict__ shared_out,
                                   T* __restrict__ out, int width, int top, size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t token = e / width;
        const int column = (int)(e % width);
        float sum = 0.0f;
        for (int j = 0; j < top; ++j)
            sum = fmaf(weights[token * top + j], down[(token * top + j) * width + column], sum);
        if (shared_out) sum += Num<T>::load(shared_out + e);
        Num<T>::store(out + e, sum);
    }
}

// out[n, i] = act(gate_up[n, i], gate_up[n, I + i]) for a dense gated feed-forward with the same activation.
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int intermediate, size_t total,
                                   float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t row = e / intermediate;
        const int column = (int)(e % intermediate);
        const T* src = gate_up + row * 2 * (size_t)intermediate + column;
        Num<T>::store(out + e, gated_activation(Num<T>::load(src), Num<T>::load(src + intermediate), limit, alpha));
    }
}

// The same, eight outputs per thread with 16-byte accesses (intermediate sizes that are a multiple of 8; the hardware
// exponential and a fast division for 16-bit activations, whose rounding is far coarser than theirs).
template <typename T>
__global__ void clamped_glu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int intermediate, size_t chunks,
                                       float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    const int per_row = intermediate / 8;
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (size_t)gridDim.x * blockDim.x) {
        const size_t row = c / per_row;
        const int column = (int)(c % per_row) * 8;
        const T* src = gate_up + row * 2 * (size_t)intermediate + column;
        float gate[8], up[8], result[8];
        load8<T>(src, gate);
        load8<T>(src + intermediate, up);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (sizeof(T) == 2) {
                const float g = fminf(gate[j], limit);
                const float u = fminf(fmaxf(up[j], -limit), limit);
                result[j] = __fdividef(g, 1.0f + __expf(-alpha * g)) * (u + 1.0f);
            } else {
                result[j] = gated_activation(gate[j], up[j], limit, alpha);
            }
        }
        store8<T>(out + row * (size_t)intermediate + column, result);
    }
}

LLM_EXPORT int llm_moe_route(const void* x, const float* router, const float* correction, int* chosen, float* weights,
                             int* counts, int n_tokens, int width, int experts, int top, float scale, int dtype,
                             cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (top <= 0 || top > experts || top > MOE_MAX_TOP) {
        llm_set_error("moe_route: top %d must lie in 1..min(%d experts, %d)", top, experts, MOE_MAX_TOP);
        return LLM_REFUSED;
    }
    const size_t shared = ((size_t)width + 2 * (size_t)experts) * sizeof(float);
    if (shared > 200 * 1024) {
        llm_set_error("moe_route: width %d and %d experts need %zu bytes of shared memory", width, experts, shared);
        return LLM_REFUSED;
    }
    LLM_DISPATCH_DTYPE(dtype, {
        if (shared > 48 * 1024) {
            const int status = llm_raise_shared_limit((const void*)moe_route_kernel<T>, shared, "moe_route");
            if (status != LLM_OK) return status;
        }
        llm_launch(moe_route_kernel<T>, n_tokens, 256, shared, stream, (const T*)x, router, correction, chosen, weights,
                   counts, width, experts, top, scale);
    });
    return llm_check_launch("moe_route");
}

LLM_EXPORT int llm_moe_select(const float* logits, const float* correction, int* chosen, float* weights, int n_tokens,
                              int experts, int top, float scale, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (top <= 0 || top > experts || top > MOE_MAX_TOP) {
        llm_set_error("moe_select: top %d must lie in 1..min(%d experts, %d)", top, experts, MOE_MAX_TOP);
        return LLM_REFUSED;
    }
    const int warps = 4;
    const size_t shared = (size_t)warps * 2 * experts * sizeof(float);
    if (shared > 40 * 1024) {
        llm_set_error("moe_select: %d experts are too many", experts);
        return LLM_REFUSED;
    }
    llm_launch(moe_select_kernel, (n_tokens + warps - 1) / warps, warps * 32, shared, stream, logits, correction, chosen, weights,
               n_tokens, experts, top, scale);
    return llm_check_launch("moe_select");
}

LLM_EXPORT int llm_indexed_linear(const void* in, const void* weight, const int* index, void* out, int n_pairs, int rows,
                                  int inner, int in_div, int gated, float limit, float alpha, int dtype, int out_f32,
                                  int index_mod, const float* in_scale, float up_shift, cudaStream_t stream) {
    if (n_pairs == 0 || rows == 0) return LLM_OK;
    if (in_div <= 0 || inner <= 0) {
        llm_set_error("indexed_linear: in_div %d and inner %d must be positive", in_div, inner);
        return LLM_REFUSED;
    }
    const size_t shared = (size_t)inner * sizeof(float);
    if (shared > 200 * 1024) {
        llm_set_error("indexed_linear: an inner size of %d needs %zu bytes of shared memory", inner, shared);
        return LLM_REFUSED;
    }
    const int warps = 8;
    dim3 grid(n_pairs, (rows + warps * 4 - 1) / (warps * 4));
    if (grid.y > 65535) {
        llm_set_error("indexed_linear: %d output elements per pair are too many for one launch", rows);
        return LLM_REFUSED;
    }
#define LLM_INDEXED(O, GATED)                                                                                           \
    do {                                                                                                                \
        if (shared > 48 * 1024) {                                                                                       \
            const int status = llm_raise_shared_limit((const void*)indexed_linear_kernel<T, O, GATED>, shared, "indexed_linear"); \
            if (status != LLM_OK) return status;                                                                        \
        }                                                                                                               \
        llm_launch(indexed_linear_kernel<T, O, GATED>, grid, warps * 32, shared, stream, (const T*)in, (const T*)weight, index, \
                   (O*)out, rows, inner, in_div, limit, alpha, index_mod, in_scale, up_shift);                                  \
    } while (0)
    LLM_DISPATCH_DTYPE(dtype, {
        if (gated && out_f32) {
            llm_set_error("indexed_linear: the gated form writes the activation type");
            return LLM_REFUSED;
        }
        if (gated) LLM_INDEXED(T, true);
        else if (out_f32) LLM_INDEXED(float, false);
        else LLM_INDEXED(T, false);
    });
#undef LLM_INDEXED
    return llm_check_launch("indexed_linear");
}

LLM_EXPORT int llm_moe_combine(const float* down, const float* weights, const void* shared_out, void* out, int n_tokens,
                               int width, int top, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    const size_t total = (size_t)n_tokens * width;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(moe_combine_kernel<T>, (unsigned)blocks, 256, 0, stream, down, weights,
                                  (const T*)shared_out, (T*)out, width, top, total)));
    return llm_check_launch("moe_combine");
}

LLM_EXPORT int llm_clamped_glu(const void* gate_up, void* out, int n_rows, int intermediate, float limit, float alpha,
                               int dtype, cudaStream_t stream) {
    if (n_rows == 0 || intermediate == 0) return LLM_OK;
    const size_t total = (size_t)n_rows * intermediate;
    if (intermediate % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
        const size_t chunks = total / 8;
        size_t vec_blocks = (chunks + 255) / 256;
        if (vec_blocks > 148 * 16) vec_blocks = 148 * 16;
        LLM_DISPATCH_DTYPE(dtype, (llm_launch(clamped_glu_vec_kernel<T>, (unsigned)vec_blocks, 256, 0, stream, (const T*)gate_up,
                                      (T*)out, intermediate, chunks, limit, alpha)));
        return llm_check_launch("clamped_glu");
    }
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(clamped_glu_kernel<T>, (unsigned)blocks, 256, 0, stream, (const T*)gate_up, (T*)out,
                                  intermediate, total, limit, alpha)));
    return llm_check_launch("clamped_glu");
}
