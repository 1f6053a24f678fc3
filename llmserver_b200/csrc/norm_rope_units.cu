// Bias + per-unit RMSNorm + rotary positions + paged K/V write for projections whose heads are made of several
// units, with query units, key units and value heads of three different sizes.
//
// The packed projection of a token is [Hq * M * Dq | Hkv * M * Dk | Hkv * Dv | ...]: every query head and every key
// head consists of M units ("maps": a head that attends with several score maps has one query and one key unit per
// map; M = 1 is the ordinary head).  Columns behind the values are left alone.  One warp per (token, unit):
//   1. the unit's elements, plus the projection's bias where there is one, in 32-bit;
//   2. RMSNorm over the unit with a weight shared by all units of its kind (`q_weight` [Dq], `k_weight` [Dk]); with
//      `k_norm_dim` > 0 only the first `k_norm_dim` elements of a key unit are normalised (among themselves) and the
//      rest stays as projected: a latent with a positional part behind it;
//   2b. query units multiplied by a factor that grows with the position p,
//        1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)                      (temp_every 0: no factor);
//   3. `rotary_dim` elements rotated, from element `q_rot_start` / `k_rot_start` of the unit on (negative: units of
//      that kind do not rotate), element i paired with i + rotary_dim / 2 or, `interleaved`, 2i with 2i + 1:
//        (u, v) -> (u cos a - v sin a, v cos a + u sin a),  a = position * inv_freq[i];
//   4. query units written back where they lie, or packed into `q_out` [N, Hq * M * Dq]; key units written into
//      the token's slot of the K pages [page, Hkv, slot, M * Dk]; value heads (bias added) into the V pages
//      [page, Hkv, slot, Dv].
// Each of bias, norms, rotation and values may be absent (Dv = 0: a cache of keys alone, as for a latent that serves as
// key and value).  Sums, angles and products are 32-bit; every element is rounded once, when it is stored.
#include "common.cuh"

template <typename T, typename W>
__global__ void norm_rope_units_kernel(T* __restrict__ qkv, int row_width, const float* __restrict__ bias,
                                       const W* __restrict__ q_weight, const W* __restrict__ k_weight, float eps,
                                       const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                       const int* __restrict__ seq_of_token, const int* __restrict__ block_tables,
                                       int max_blocks, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                       int n_q_heads, int n_kv_heads, int maps, int q_dim, int k_dim, int value_dim,
                                       int page_size, int num_pages, int write_cache, int* __restrict__ error_flag,
                                       int rotary_dim, int max_dim, int k_norm_dim, int q_rot_start, int k_rot_start,
                                       int interleaved, float temp_coef, int temp_every) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float unit_values[];     // [warps][max_dim]
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    float* values = unit_values + (size_t)warp * max_dim;
    const int position = positions[token];
    const int half = rotary_dim >> 1;
    // the token's cosines and sines, made once for all of its units
    float2* rotation = reinterpret_cast<float2*>(unit_values + (size_t)warps * max_dim);
    if (inv_freq) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float angle = (float)position * inv_freq[i];
            rotation[i] = make_float2(cosf(angle), sinf(angle));
        }
        __syncthreads();
    }
    const int q_units = n_q_heads * maps, k_units = n_kv_heads * maps;
    const int total_units = q_units + k_units + (value_dim > 0 ? n_kv_heads : 0);
    T* row = qkv + (size_t)token * row_width;
    for (int unit = blockIdx.y * warps + warp; unit < total_units; unit += gridDim.y * warps) {
        const bool is_q = unit < q_units;
        const bool is_k = !is_q && unit < q_units + k_units;
        int dim, column;
        if (is_q) {
            dim = q_dim;
            column = unit * q_dim;
        } else if (is_k) {
            dim = k_dim;
            column = q_units * q_dim + (unit - q_units) * k_dim;
        } else {
            dim = value_dim;
            column = q_units * q_dim + k_units * k_dim + (unit - q_units - k_units) * value_dim;
        }
        T* dst;
        if (is_q) {
            dst = q_out ? q_out + (size_t)token * q_units * q_dim + (size_t)unit * q_dim : row + column;
        } else {
            if (!write_cache) continue;
            const int page = block_tables[(size_t)seq_of_token[token] * max_blocks + position / page_size];
            if (page < 0 || page >= num_pages) {
                if (lane == 0) atomicExch(error_flag, 1 + token);   // the host turns this into an exception
                continue;
            }
            if (is_k) {
                const int k_unit = unit - q_units;
                const size_t slot = ((size_t)page * n_kv_heads + k_unit / maps) * page_size + position % page_size;
                dst = k_pages + slot * ((size_t)maps * k_dim) + (size_t)(k_unit % maps) * k_dim;
            } else {
                const size_t slot = ((size_t)page * n_kv_heads + (unit - q_units - k_units)) * page_size + position % page_size;
                dst = v_pages + slot * value_dim;
            }
        }
        const int norm_dim = (is_k && k_norm_dim > 0) ? k_norm_dim : dim;
        const W* weight = is_q ? q_weight : (is_k ? k_weight : nullptr);
        const int rot_start = is_q ? q_rot_start : (is_k ? k_rot_start : -1);
        const int turning = (inv_freq && rot_start >= 0) ? rotary_dim : 0;
        // a query unit that stays where it lies and only turns: nothing but its turning elements is read or written
        const bool only_turns = is_q && !q_out && !weight && !bias && temp_every <= 0;
        const int from = only_turns ? rot_start : 0, upto = only_turns ? rot_start + turning : dim;
        float sum_squares = 0.0f;
        for (int i = from + lane; i < upto; i += 32) {
            float v = Num<T>::load(row + column + i);
            if (bias) v += bias[column + i];
            values[i] = v;
            if (i < norm_dim) sum_squares += v * v;
        }
        if (weight) {
            const float inverse = rsqrtf(warp_sum(sum_squares) / (float)norm_dim + eps);
            for (int i = lane; i < norm_dim; i += 32) values[i] = values[i] * inverse * Num<W>::load(weight + i);
        }
        if (is_q && temp_every > 0) {
            const float factor = 1.0f + temp_coef * logf((float)((position + 1) / temp_every) + 1.0f);
            for (int i = lane; i < dim; i += 32) values[i] *= factor;
        }
        __syncwarp();
        for (int i = lane; i < turning / 2; i += 32) {
            const float c = rotation[i].x, s = rotation[i].y;
            const int first = rot_start + (interleaved ? 2 * i : i), second = interleaved ? first + 1 : first + half;
            const float u = values[first], v = values[second];
            Num<T>::store(dst + first, u * c - v * s);
            Num<T>::store(dst + second, v * c + u * s);
        }
        if (!only_turns)
            for (int i = lane; i < dim; i += 32)
                if (turning == 0 || i < rot_start || i >= rot_start + turning) Num<T>::store(dst + i, values[i]);
        __syncwarp();      // the next unit of this warp overwrites the values
    }
}

LLM_EXPORT int llm_norm_rope_units(void* qkv, int row_width, const float* bias, const void* q_weight, const void* k_weight,
                                   float eps, const float* inv_freq, const int* positions, const int* seq_of_token,
                                   const int* block_tables, int max_blocks, void* q_out, void* k_pages, void* v_pages,
                                   int n_tokens, int n_q_heads, int n_kv_heads, int maps, int q_dim, int k_dim, int value_dim,
                                   int page_size, int num_pages, int write_cache, int* error_flag, int rotary_dim, int dtype,
                                   int weight_dtype, int k_norm_dim, int q_rot_start, int k_rot_start, int interleaved,
                                   float temp_coef, int temp_every, cudaStream_t stream) {
    if (n_tokens == 0) return LLM_OK;
    if (inv_freq == nullptr) rotary_dim = 0;
    if (n_kv_heads == 0) {      // queries alone: nothing is cached
        k_dim = k_dim > 0 ? k_dim : 1;
        page_size = num_pages = 1;
        value_dim = 0;
        if (k_rot_start >= 0) k_rot_start = -1;
    }
    if (n_q_heads <= 0 || n_kv_heads < 0 || maps <= 0 || q_dim <= 0 || k_dim <= 0 || value_dim < 0 || page_size <= 0 || num_pages <= 0) {
        llm_set_error("norm_rope_units: sizes must be positive (value_dim and the key heads may be 0)");
        return LLM_REFUSED;
    }
    if (rotary_dim < 0 || rotary_dim % 2 || (q_rot_start >= 0 && q_rot_start + rotary_dim > q_dim) ||
        (k_rot_start >= 0 && k_rot_start + rotary_dim > k_dim)) {
        llm_set_error("norm_rope_units: %d rotating elements from %d / %d must be an even number inside units of %d and %d",
                      rotary_dim, q_rot_start, k_rot_start, q_dim, k_dim);
        return LLM_REFUSED;
    }
    if (k_norm_dim < 0 || k_norm_dim > k_dim || temp_every < 0) {
        llm_set_error("norm_rope_units: a key unit of %d cannot normalise %d elements (or the temperature's period %d is negative)",
                      k_dim, k_norm_dim, temp_every);
        return LLM_REFUSED;
    }
    const long long used = (long long)(n_q_heads * maps) * q_dim + (long long)(n_kv_heads * maps) * k_dim + (long long)n_kv_heads * value_dim;
    if (row_width < used) {
        llm_set_error("norm_rope_units: rows of %d columns cannot hold %lld", row_width, used);
        return LLM_REFUSED;
    }
    int max_dim = q_dim > k_dim ? q_dim : k_dim;
    if (value_dim > max_dim) max_dim = value_dim;
    const int warps = 4;
    const size_t shared = (size_t)warps * max_dim * sizeof(float) + (size_t)(rotary_dim / 2 + 1) * sizeof(float2);
    if (shared > 160 * 1024) {
        llm_set_error("norm_rope_units: units of %d elements need %zu bytes of shared memory", max_dim, shared);
        return LLM_REFUSED;
    }
    const int total_units = (n_q_heads + n_kv_heads) * maps + (value_dim > 0 ? n_kv_heads : 0);
    int slices = (total_units + warps - 1) / warps;
    if (n_tokens >= 1024 && slices > 2) slices = 2;      // long prompts: fewer, longer-lived blocks
    dim3 grid(n_tokens, slices);
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, {
        if (shared > 40 * 1024) {
            const int status = llm_raise_shared_limit((const void*)norm_rope_units_kernel<T, W>, shared, "norm_rope_units");
            if (status != LLM_OK) return status;
        }
        llm_launch(norm_rope_units_kernel<T, W>, grid, warps * 32, shared, stream, (T*)qkv, row_width, bias, (const W*)q_weight,
                   (const W*)k_weight, eps, inv_freq, positions, seq_of_token, block_tables, max_blocks, (T*)q_out, (T*)k_pages,
                   (T*)v_pages, n_q_heads, n_kv_heads, maps, q_dim, k_dim, value_dim, page_size, num_pages, write_cache, error_flag,
                   rotary_dim, max_dim, k_norm_dim, q_rot_start, k_rot_start, interleaved, temp_coef, temp_every);
    });
    return llm_check_launch("norm_rope_units");
}
