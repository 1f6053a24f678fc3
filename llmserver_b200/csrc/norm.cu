// RMSNorm and residual-add + RMSNorm over the 32-bit residual stream.
//
//   residual[r] += delta[r]            (32-bit sum; skipped when delta is null)
//   out[o]       = residual[r] * rsqrt(mean(residual[r]^2) + eps) * weight
//
// Statistics, the product with the weight and the residual sum are 32-bit; the result is rounded
// once to the activation type.  The reference's fused kernel (utils/fused_ops.py:65-78) rounds
// the residual sum to the activation type first; keeping the stream in 32-bit is more exact.
// `rows` (optional) selects the source rows: output row o reads row rows[o]; used for the final
// norm, which runs only where logits are wanted (utils/model.py:147-157).
// With `squares_out` the division by the root mean square is left to the consumer: out = residual * weight, and
// squares_out[o] = sum(residual[r]^2), for a product kernel that scales its accumulators row by row.
//
// Two forms of the same arithmetic: a vector form (16-byte accesses, the row held in registers between
// the two passes) for widths that are a multiple of 8 and at most 16384, and a scalar form for the rest.
// The sum of squares is taken in the same order in both passes of a form, and the order depends on the
// width only, never on how many rows the call has.
#include "common.cuh"

namespace {
constexpr int kChunk = 8;        // elements a thread handles at a time in the vector form
constexpr int kMaxChunks = 4;    // per thread
}

template <typename T, typename W>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const W* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ rows, int width, float eps, int write_residual,
                                       float* __restrict__ squares_out) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    __shared__ float scratch[33];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* res = residual + (size_t)r * width;
    const T* del = delta ? delta + (size_t)r * width : nullptr;
    const int chunks = width / kChunk;
    float values[kMaxChunks][kChunk];
    float sum_squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            load8<float>(res + c * kChunk, values[i]);
            if (del) {
                float added[kChunk];
                load8<T>(del + c * kChunk, added);
#pragma unroll
                for (int j = 0; j < kChunk; ++j) values[i][j] += added[j];
                if (write_residual) store8<float>(res + c * kChunk, values[i]);
            }
#pragma unroll
            for (int j = 0; j < kChunk; ++j) sum_squares += values[i][j] * values[i][j];
        }
    }
    const float total = block_sum(sum_squares, scratch);
    const float inverse = squares_out ? 1.0f : rsqrtf(total / (float)width + eps);
    if (squares_out && threadIdx.x == 0) squares_out[o] = total;
    T* dst = out + (size_t)o * width;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            float scale[kChunk], scaled[kChunk];
            load8<W>(weight + c * kChunk, scale);
#pragma unroll
            for (int j = 0; j < kChunk; ++j) scaled[j] = values[i][j] * inverse * scale[j];
            store8<T>(dst + c * kChunk, scaled);
        }
    }
}

template <typename T, typename W>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const W* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps, int write_residual,
                                       float* __restrict__ squares_out) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    __shared__ float scratch[33];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* res = residual + (size_t)r * width;
    const T* del = delta ? delta + (size_t)r * width : nullptr;
    float sum_squares = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (del) {
            v += Num<T>::load(del + i);
            if (write_residual) res[i] = v;
        }
        sum_squares += v * v;
    }
    const float total = block_sum(sum_squares, scratch);
    const float inverse = squares_out ? 1.0f : rsqrtf(total / (float)width + eps);
    if (squares_out && threadIdx.x == 0) squares_out[o] = total;
    T* dst = out + (size_t)o * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (del && !write_residual) v += Num<T>::load(del + i);
        Num<T>::store(dst + i, v * inverse * Num<W>::load(weight + i));
    }
}

// Plain RMSNorm of activation-typed rows (used by parts that normalise something other than the
// residual stream).  Same arithmetic.
template <typename T, typename W>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const W* __restrict__ weight, T* __restrict__ out,
                               int width, float eps) {
    pdl_trigger();   // let the next kernel start launching
    pdl_wait();      // everything before this kernel in the stream is complete and visible
    __shared__ float scratch[33];
    const T* src = x + (size_t)blockIdx.x * width;
    float sum_squares = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = Num<T>::load(src + i);
        sum_squares += v * v;
    }
    const float total = block_sum(sum_squares, scratch);
    const float inverse = rsqrtf(total / (float)width + eps);
    T* dst = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        Num<T>::store(dst + i, Num<T>::load(src + i) * inverse * Num<W>::load(weight + i));
}

static int norm_threads(int width) { return width >= 2048 ? 512 : (width >= 512 ? 256 : 128); }

LLM_EXPORT int llm_add_rmsnorm(float* residual, const void* delta, const void* weight, void* out, const int* rows,
                               int n_rows, int width, float eps, int write_residual, int dtype,
                               int weight_dtype, float* squares_out, cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    const int chunks = width / kChunk;
    // the block size depends on the width only, so a row is summed in the same order in every call
    int threads = ((chunks + 31) / 32) * 32;
    if (threads > 512) threads = 512;
    const bool vector_form = width % kChunk == 0 && width >= kChunk && aligned16(residual) && aligned16(out) &&
                             aligned16(delta) && aligned16(weight) && chunks <= threads * kMaxChunks;
    if (vector_form) {
        LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype,
                                  (llm_launch(add_rmsnorm_vec_kernel<T, W>, n_rows, threads, 0, stream, 
                                      residual, (const T*)delta, (const W*)weight, (T*)out, rows, width, eps,
                                      write_residual, squares_out)));
        return llm_check_launch("add_rmsnorm");
    }
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype,
                              (llm_launch(add_rmsnorm_kernel<T, W>, n_rows, norm_threads(width), 0, stream, 
                                  residual, (const T*)delta, (const W*)weight, (T*)out, rows, width, eps,
                                  write_residual, squares_out)));
    return llm_check_launch("add_rmsnorm");
}

LLM_EXPORT int llm_rmsnorm(const void* x, const void* weight, void* out, int n_rows, int width, float eps,
                           int dtype, int weight_dtype, cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype,
                              (llm_launch(rmsnorm_kernel<T, W>, n_rows, norm_threads(width), 0, stream, 
                                  (const T*)x, (const W*)weight, (T*)out, width, eps)));
    return llm_check_launch("rmsnorm");
}

// A sub-layer whose output is normalised before it joins the stream, fused with the norm that follows:
//   residual[r] += d * rsqrt(mean(d^2) + post_eps) * post_weight (+ extra[r]),  d = delta[r] (+ delta_bias)
//   out[o]       = residual[r] * rsqrt(mean(residual[r]^2) + eps) * weight          (skipped when out is null)
// `delta_bias` (32-bit, [width]) is the bias of the projection that made delta, added here in 32-bit.  Without `weight`
// the output is the updated stream itself in the activation type: what a sub-layer reads that takes the stream as it is.
// `extra` is a second 32-bit stream added at the same time (a model that feeds its embedding in again).  Both
// statistics, both products and the sum are 32-bit; the updated row waits in shared memory between the passes.
template <typename T, typename W>
__global__ void normed_add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                          const W* __restrict__ post_weight, float post_eps, const float* __restrict__ extra,
                                          const W* __restrict__ weight, T* __restrict__ out, const int* __restrict__ rows,
                                          int width, float eps, int write_residual, const float* __restrict__ delta_bias) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    extern __shared__ float updated[];     // [width]
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* res = residual + (size_t)r * width;
    float inverse_post = 0.0f;
    if (delta) {
        const T* del = delta + (size_t)r * width;
        float sum_squares = 0.0f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = Num<T>::load(del + i) + (delta_bias ? delta_bias[i] : 0.0f);
            updated[i] = v;
            sum_squares += v * v;
        }
        inverse_post = rsqrtf(block_sum(sum_squares, scratch) / (float)width + post_eps);
    }
    float sum_squares = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (delta) v += updated[i] * inverse_post * Num<W>::load(post_weight + i);
        if (extra) v += extra[(size_t)r * width + i];
        if (write_residual && (delta || extra)) res[i] = v;
        updated[i] = v;
        sum_squares += v * v;
    }
    if (!out) return;
    T* dst = out + (size_t)o * width;
    if (!weight) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) Num<T>::store(dst + i, updated[i]);
        return;
    }
    const float inverse = rsqrtf(block_sum(sum_squares, scratch) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        Num<T>::store(dst + i, updated[i] * inverse * Num<W>::load(weight + i));
}

// The same with 16-byte accesses and the row held in registers between the passes (widths that are a multiple of 8,
// up to blockDim * 32); the order of each sum depends on the width only.
template <typename T, typename W>
__global__ void normed_add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                              const W* __restrict__ post_weight, float post_eps, const float* __restrict__ extra,
                                              const W* __restrict__ weight, T* __restrict__ out, const int* __restrict__ rows,
                                              int width, float eps, int write_residual, const float* __restrict__ delta_bias) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* res = residual + (size_t)r * width;
    const int chunks = width / kChunk;
    float values[kMaxChunks][kChunk];
    float inverse_post = 0.0f;
    if (delta) {
        const T* del = delta + (size_t)r * width;
        float sum_squares = 0.0f;
#pragma unroll
        for (int i = 0; i < kMaxChunks; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < chunks) {
                load8<T>(del + c * kChunk, values[i]);
                if (delta_bias) {
                    float bias[kChunk];
                    load8<float>(delta_bias + c * kChunk, bias);
#pragma unroll
                    for (int j = 0; j < kChunk; ++j) values[i][j] += bias[j];
                }
#pragma unroll
                for (int j = 0; j < kChunk; ++j) sum_squares += values[i][j] * values[i][j];
            }
        }
        inverse_post = rsqrtf(block_sum(sum_squares, scratch) / (float)width + post_eps);
    }
    float sum_squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            float stream[kChunk];
            load8<float>(res + c * kChunk, stream);
            if (delta) {
                float scale[kChunk];
                load8<W>(post_weight + c * kChunk, scale);
#pragma unroll
                for (int j = 0; j < kChunk; ++j) stream[j] += values[i][j] * inverse_post * scale[j];
            }
            if (extra) {
                float more[kChunk];
                load8<float>(extra + (size_t)r * width + c * kChunk, more);
#pragma unroll
                for (int j = 0; j < kChunk; ++j) stream[j] += more[j];
            }
            if (write_residual && (delta || extra)) store8<float>(res + c * kChunk, stream);
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
                values[i][j] = stream[j];
                sum_squares += stream[j] * stream[j];
            }
        }
    }
    if (!out) return;
    T* dst = out + (size_t)o * width;
    if (!weight) {
#pragma unroll
        for (int i = 0; i < kMaxChunks; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < chunks) store8<T>(dst + c * kChunk, values[i]);
        }
        return;
    }
    const float inverse = rsqrtf(block_sum(sum_squares, scratch) / (float)width + eps);
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            float scale[kChunk], scaled[kChunk];
            load8<W>(weight + c * kChunk, scale);
#pragma unroll
            for (int j = 0; j < kChunk; ++j) scaled[j] = values[i][j] * inverse * scale[j];
            store8<T>(dst + c * kChunk, scaled);
        }
    }
}

LLM_EXPORT int llm_normed_add_rmsnorm(float* residual, const void* delta, const void* post_weight, float post_eps,
                                      const float* extra, const void* weight, void* out, const int* rows, int n_rows,
                                      int width, float eps, int write_residual, int dtype, int weight_dtype,
                                      const float* delta_bias, cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    if (delta && !post_weight) {
        llm_set_error("normed_add_rmsnorm: a delta needs the weight of its norm");
        return LLM_REFUSED;
    }
    const int chunks = width / kChunk;
    int threads = ((chunks + 31) / 32) * 32;      // depends on the width only
    if (threads > 512) threads = 512;
    const bool vector_form = width % kChunk == 0 && width >= kChunk && chunks <= threads * kMaxChunks && aligned16(residual) &&
                             aligned16(delta) && aligned16(post_weight) && aligned16(extra) && aligned16(weight) && aligned16(out) && aligned16(delta_bias);
    if (vector_form) {
        LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype,
                                  (llm_launch(normed_add_rmsnorm_vec_kernel<T, W>, n_rows, threads, 0, stream, residual,
                                      (const T*)delta, (const W*)post_weight, post_eps, extra, (const W*)weight, (T*)out, rows,
                                      width, eps, write_residual, delta_bias)));
        return llm_check_launch("normed_add_rmsnorm");
    }
    const size_t shared = (size_t)width * sizeof(float);
    if (shared > 200 * 1024) {
        llm_set_error("normed_add_rmsnorm: a width of %d needs %zu bytes of shared memory", width, shared);
        return LLM_REFUSED;
    }
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, {
        if (shared > 40 * 1024) {
            const int status = llm_raise_shared_limit((const void*)normed_add_rmsnorm_kernel<T, W>, shared + 256, "normed_add_rmsnorm");
            if (status != LLM_OK) return status;
        }
        llm_launch(normed_add_rmsnorm_kernel<T, W>, n_rows, norm_threads(width), shared, stream, residual, (const T*)delta,
                   (const W*)post_weight, post_eps, extra, (const W*)weight, (T*)out, rows, width, eps, write_residual, delta_bias);
    });
    return llm_check_launch("normed_add_rmsnorm");
}

// Two sub-layers that read the same normalised stream and join it together, each through a learned scale per channel,
// fused with the norm that follows:
//   residual[r] += a[r] * scale_a (+ b[r] * scale_b)        (32-bit products and sums; scales are 32-bit [width])
//   out[o]       = residual[r] * rsqrt(mean(residual[r]^2) + eps) * weight          (skipped when out is null)
// `b` may be absent (a layer without its second sub-layer).  With `rows` the stream is left as it was.
template <typename T, typename W>
__global__ void scaled_add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ a, const float* __restrict__ scale_a,
                                          const T* __restrict__ b, const float* __restrict__ scale_b, const W* __restrict__ weight,
                                          T* __restrict__ out, const int* __restrict__ rows, int width, float eps, int write_residual) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    extern __shared__ float updated[];     // [width]
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* res = residual + (size_t)r * width;
    float sum_squares = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        float added = Num<T>::load(a + (size_t)r * width + i) * scale_a[i];
        if (b) added = fmaf(Num<T>::load(b + (size_t)r * width + i), scale_b[i], added);
        v += added;
        if (write_residual) res[i] = v;
        updated[i] = v;
        sum_squares += v * v;
    }
    if (!out) return;
    const float inverse = rsqrtf(block_sum(sum_squares, scratch) / (float)width + eps);
    T* dst = out + (size_t)o * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        Num<T>::store(dst + i, updated[i] * inverse * Num<W>::load(weight + i));
}

// The same with 16-byte accesses and the row held in registers between the passes; sums in the scalar form's order per
// element, the sum of squares in an order that depends on the width only.
template <typename T, typename W>
__global__ void scaled_add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ a, const float* __restrict__ scale_a,
                                              const T* __restrict__ b, const float* __restrict__ scale_b, const W* __restrict__ weight,
                                              T* __restrict__ out, const int* __restrict__ rows, int width, float eps,
                                              int write_residual) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* res = residual + (size_t)r * width;
    const int chunks = width / kChunk;
    float values[kMaxChunks][kChunk];
    float sum_squares = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            float part[kChunk], scale[kChunk], added[kChunk];
            load8<float>(res + c * kChunk, values[i]);
            load8<T>(a + (size_t)r * width + c * kChunk, part);
            load8<float>(scale_a + c * kChunk, scale);
#pragma unroll
            for (int j = 0; j < kChunk; ++j) added[j] = part[j] * scale[j];
            if (b) {
                load8<T>(b + (size_t)r * width + c * kChunk, part);
                load8<float>(scale_b + c * kChunk, scale);
#pragma unroll
                for (int j = 0; j < kChunk; ++j) added[j] = fmaf(part[j], scale[j], added[j]);
            }
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
                values[i][j] += added[j];
                sum_squares += values[i][j] * values[i][j];
            }
            if (write_residual) store8<float>(res + c * kChunk, values[i]);
        }
    }
    if (!out) return;
    const float inverse = rsqrtf(block_sum(sum_squares, scratch) / (float)width + eps);
    T* dst = out + (size_t)o * width;
#pragma unroll
    for (int i = 0; i < kMaxChunks; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < chunks) {
            float scale[kChunk], scaled[kChunk];
            load8<W>(weight + c * kChunk, scale);
#pragma unroll
            for (int j = 0; j < kChunk; ++j) scaled[j] = values[i][j] * inverse * scale[j];
            store8<T>(dst + c * kChunk, scaled);
        }
    }
}

LLM_EXPORT int llm_scaled_add_rmsnorm(float* residual, const void* a, const float* scale_a, const void* b, const float* scale_b,
                                      const void* weight, void* out, const int* rows, int n_rows, int width, float eps,
                                      int write_residual, int dtype, int weight_dtype, cudaStream_t stream) {
    if (n_rows == 0) return LLM_OK;
    if (!a || !scale_a || (b && !scale_b) || (out && !weight)) {
        llm_set_error("scaled_add_rmsnorm: a sub-layer output needs its scale, an output the norm's weight");
        return LLM_REFUSED;
    }
    const int chunks = width / kChunk;
    int threads = ((chunks + 31) / 32) * 32;      // depends on the width only
    if (threads > 512) threads = 512;
    const bool vector_form = width % kChunk == 0 && width >= kChunk && chunks <= threads * kMaxChunks && aligned16(residual) &&
                             aligned16(a) && aligned16(b) && aligned16(scale_a) && aligned16(scale_b) && aligned16(weight) && aligned16(out);
    if (vector_form) {
        LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype,
                                  (llm_launch(scaled_add_rmsnorm_vec_kernel<T, W>, n_rows, threads, 0, stream, residual, (const T*)a,
                                      scale_a, (const T*)b, scale_b, (const W*)weight, (T*)out, rows, width, eps, write_residual)));
        return llm_check_launch("scaled_add_rmsnorm");
    }
    const size_t shared = (size_t)width * sizeof(float);
    if (shared > 200 * 1024) {
        llm_set_error("scaled_add_rmsnorm: a width of %d needs %zu bytes of shared memory", width, shared);
        return LLM_REFUSED;
    }
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, {
        if (shared > 40 * 1024) {
            const int status = llm_raise_shared_limit((const void*)scaled_add_rmsnorm_kernel<T, W>, shared + 256, "scaled_add_rmsnorm");
            if (status != LLM_OK) return status;
        }
        llm_launch(scaled_add_rmsnorm_kernel<T, W>, n_rows, norm_threads(width), shared, stream, residual, (const T*)a, scale_a,
                   (const T*)b, scale_b, (const W*)weight, (T*)out, rows, width, eps, write_residual);
    });
    return llm_check_launch("scaled_add_rmsnorm");
}
