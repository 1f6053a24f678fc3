// Recurrences with a matrix-valued state per head, kept in 32-bit per request, and what surrounds them: the mix of
// each token with the one before it, short causal convolutions over time, and the head norm and output gate.
//
// (1) Token shift (`llm_token_shift_mix`): with h' the row of the token before (the sequence's stored row for the first
//     token of a step, zeros for the first token of a sequence), out[s] = h + (h' - h) * mu[s] for each of M mixing
//     vectors.  The stored row is replaced by the kernel of (3), behind every read of it.
//
// (2) Short convolution (`llm_short_conv_units`): y_t[c] = silu(sum_j w[c][j] * x_(t - taps + 1 + j)[c]), zeros before the
//     sequence's start, the last taps - 1 inputs of every sequence carried in its state slot; channels come in units (a
//     head's query, key or value channels); the first `n_unit_norm` units are then made unit vectors,
//     y / sqrt(sum(y^2) + norm_eps), and the first `n_scaled` of those multiplied by `scale`.  Results are 32-bit.  A block
//     takes 64 tokens of one unit; only a sequence's first block touches its stored inputs (a chunk is longer than any
//     history), reads them for its first tokens and then brings them up to date.
//
// (3) The recurrences (`llm_wkv_recurrent`, `llm_delta_rule_recurrent`), per head with S in R^(dim x vdim):
//       wkv     o_t = (S + diag(u) k_t v_t^T)^T r_t;   S <- diag(w_t) S + k_t v_t^T;   w_t = exp(-exp(z_t + w0))
//       delta   S <- g_t S;  d = beta_t (v_t - S^T k_t);  S <- S + k_t d^T;  o_t = S^T q_t
//               g_t = exp(-exp(A) softplus(a_t + dt)),  beta_t = sigmoid(b_t)
//     followed by out = o / sqrt(mean(o^2) + eps) * weight * silu(gate).
//
// One block per (sequence, head).  A warp covers 32 / P value channels (columns of S) with P row partitions side by
// side in its lanes; a thread owns R rows of one column in registers, so a sum over the rows is R multiply-adds and
// log2(P) shuffles, with no block barrier inside the walk over tokens.  Tokens are taken sixteen at a time: staged in
// shared memory in 32-bit (decays, gates and step sizes formed there), walked on the registers, then normalised, gated
// and stored by one warp per token.  The order of every sum depends on the sizes alone, so a token's result does not
// depend on how its prompt was cut or on what else is in the batch.
//
// Long portions can also be walked segment by segment in parallel (a segment length given to the launchers).  Both
// recurrences are linear in S: behind a segment, S_out = M S_in + L, where L is what the segment leaves from a zero state
// and M its transition: diag(prod_t w_t) for wkv; for the delta rule the product of the g_t (I - beta_t k_t k_t^T), a
// dim x dim matrix, which the same walk yields column by column when it starts from the identity with values of zero.
// Pass A runs every segment but the last from zero (delta: also `dim` more columns from the identity) and leaves L and M;
// a scan gives every segment the state it starts from, S_in(k + 1) = M_k S_in(k) + L_k; pass C runs the segments again
// from those states and writes the outputs.  All of it 32-bit; sums are then grouped by segment, so results agree with
// the one-pass form to rounding, not bit for bit (the 32-bit path keeps the one-pass form).
#include "common.cuh"

#define REC_TOKENS 16

// ------------------------------------------------------------------------------------------------ token shift
template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ h, const float* __restrict__ shift_state, const int* __restrict__ state_slots,
                                       const int* __restrict__ q_start, const int* __restrict__ seq_of_token,
                                       const float* __restrict__ mu, T* __restrict__ out, int tokens, int width, int mixes) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)tokens * width;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(e / width), c = (int)(e % width);
        const int seq = seq_of_token[t];
        const float here = Num<T>::load(h + e);
        const float before = t == q_start[seq] ? shift_state[(size_t)state_slots[seq] * width + c] : Num<T>::load(h + e - width);
        for (int s = 0; s < mixes; ++s)
            Num<T>::store(out + (size_t)s * total + e, here + (before - here) * mu[(size_t)s * width + c]);
    }
}

LLM_EXPORT int llm_token_shift_mix(const void* h, const float* shift_state, const int* state_slots, const int* q_start,
                                   const int* seq_of_token, const float* mu, void* out, int tokens, int width, int mixes, int dtype,
                                   cudaStream_t stream) {
    if (tokens == 0) return LLM_OK;
    size_t blocks = ((size_t)tokens * width + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(token_shift_mix_kernel<T>, (unsigned)blocks, 256, 0, stream, (const T*)h, shift_state,
                                          state_slots, q_start, seq_of_token, mu, (T*)out, tokens, width, mixes)));
    return llm_check_launch("token_shift_mix");
}

// ------------------------------------------------------------------------------------------------ short convolution
struct ConvArgs {
    const void* x;          // [N, row_width], the channels start at column `column`
    int row_width, column;
    const float* taps_w;    // [channels, taps]
    int taps;
    float* state;           // [slots, max(taps - 1, 1), channels]: a sequence's last inputs, oldest first
    const int* state_slots;
    const int* q_start;
    float* out;             // [N, channels]
    int channels;
    int n_unit_norm, unit_dim, n_scaled;   // units 0 .. n_unit_norm - 1 have unit_dim channels and are made unit vectors
    int n_plain, plain_dim;                // the units behind them
    float norm_eps, scale;
};

#define CONV_MAX_PER_LANE 16    // a unit has at most 32 * 16 channels
#define CONV_MAX_TAPS 8
#define CONV_CHUNK 64           // tokens per block; more than CONV_MAX_TAPS - 1, so only a sequence's first block reads stored inputs

template <typename T>
__global__ void __launch_bounds__(256) short_conv_units_kernel(ConvArgs a) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x, unit = blockIdx.y;
    const int begin = a.q_start[seq], end = a.q_start[seq + 1];
    const int chunk_begin = begin + blockIdx.z * CONV_CHUNK, chunk_end = min(end, chunk_begin + CONV_CHUNK);
    if (chunk_begin >= end) return;
    const bool normed = unit < a.n_unit_norm;
    const int size = normed ? a.unit_dim : a.plain_dim;
    const int first = normed ? unit * a.unit_dim : a.n_unit_norm * a.unit_dim + (unit - a.n_unit_norm) * a.plain_dim;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int history = a.taps - 1;
    const T* x = (const T*)a.x + a.column + first;
    float* state = a.state + (size_t)a.state_slots[seq] * max(history, 1) * a.channels + first;
    for (int t = chunk_begin + warp; t < chunk_end; t += warps) {
        float y[CONV_MAX_PER_LANE];
        float squares = 0.0f;
#pragma unroll
        for (int u = 0; u < CONV_MAX_PER_LANE; ++u) {
            const int c = lane + 32 * u;
            y[u] = 0.0f;
            if (c < size) {
                float sum = 0.0f;
                for (int j = 0; j < a.taps; ++j) {
                    const int source = t - history + j;      // on the step's token axis; before `begin`: the stored inputs
                    const float value = source >= begin ? Num<T>::load(x + (size_t)source * a.row_width + c)
                                                        : state[(size_t)(history + source - begin) * a.channels + c];
                    sum = fmaf(a.taps_w[(size_t)(first + c) * a.taps + j], value, sum);
                }
                y[u] = sum / (1.0f + expf(-sum));
                squares = fmaf(y[u], y[u], squares);
            }
        }
        float factor = 1.0f;
        if (normed) {
            factor = rsqrtf(warp_sum(squares) + a.norm_eps);
            if (unit < a.n_scaled) factor *= a.scale;
        }
#pragma unroll
        for (int u = 0; u < CONV_MAX_PER_LANE; ++u) {
            const int c = lane + 32 * u;
            if (c < size) a.out[(size_t)t * a.channels + first + c] = y[u] * factor;
        }
    }
    if (blockIdx.z != 0) return;
    __syncthreads();      // every read of the stored inputs is done (they are read by this block alone)
    // the new stored inputs: the last `history` of (old stored inputs, this step's inputs); a channel is one thread's,
    // which walks its rows oldest first, so a row is read before it is overwritten
    const int length = end - begin;
    for (int c = threadIdx.x; c < size; c += blockDim.x) {
        for (int r = 0; r < history; ++r) {
            const int source = length - history + r;      // relative to `begin`
            state[(size_t)r * a.channels + c] = source >= 0 ? Num<T>::load(x + (size_t)(begin + source) * a.row_width + c)
                                                             : state[(size_t)(history + source) * a.channels + c];
        }
    }
}

LLM_EXPORT int llm_short_conv_units(const void* x, int row_width, int column, const float* taps_w, int taps, float* state,
                                    const int* state_slots, const int* q_start, float* out, int n_seqs, int longest, int n_unit_norm,
                                    int unit_dim, int n_scaled, int n_plain, int plain_dim, float norm_eps, float scale, int dtype,
                                    cudaStream_t stream) {
    if (n_seqs == 0 || longest <= 0) return LLM_OK;
    if (taps < 1 || taps > CONV_MAX_TAPS || unit_dim > 32 * CONV_MAX_PER_LANE || plain_dim > 32 * CONV_MAX_PER_LANE ||
        n_unit_norm < 0 || n_plain < 0 || n_unit_norm + n_plain == 0) {
        llm_set_error("short_conv_units: %d taps (1 to %d) over units of %d and %d channels (up to %d) are not supported", taps,
                      CONV_MAX_TAPS, unit_dim, plain_dim, 32 * CONV_MAX_PER_LANE);
        return LLM_REFUSED;
    }
    ConvArgs a;
    a.x = x; a.row_width = row_width; a.column = column; a.taps_w = taps_w; a.taps = taps; a.state = state;
    a.state_slots = state_slots; a.q_start = q_start; a.out = out;
    a.channels = n_unit_norm * unit_dim + n_plain * plain_dim;
    a.n_unit_norm = n_unit_norm; a.unit_dim = unit_dim; a.n_scaled = n_scaled; a.n_plain = n_plain; a.plain_dim = plain_dim;
    a.norm_eps = norm_eps; a.scale = scale;
    LLM_DISPATCH_DTYPE(dtype, (llm_launch(short_conv_units_kernel<T>, dim3(n_seqs, n_unit_norm + n_plain, (longest + CONV_CHUNK - 1) / CONV_CHUNK), 256, 0, stream, a)));
    return llm_check_launch("short_conv_units");
}

// ------------------------------------------------------------------------------------------------ the recurrences
struct RecArgs {
    // inputs in the activation type: a packed projection row per token
    const void* proj;
    int row_width, r_offset, k_offset, v_offset, g_offset;      // wkv: r, k, v and the gate; delta: the gate only
    // inputs in 32-bit
    const float* pre;       // delta: [N, pre_width] convolved q | k | v (q and k heads of `dim`, v heads of `vdim`)
    int pre_width, q_col, k_col, v_col, qk_heads;
    const float* wide;      // wkv: z [N, heads * dim]; delta: [N, 2 heads] = b | a
    const float* w0;        // wkv: [heads * dim]
    const float* bonus;     // wkv: u [heads, dim]
    const float* a_log;     // delta: [heads]
    const float* dt_bias;   // delta: [heads]
    const void* weight;     // norm weight, [vdim] (weight_stride 0) or [heads, vdim] (weight_stride vdim)
    int weight_stride;
    float* state;           // [slots, heads, dim, vdim]
    const int* state_slots;
    const int* q_start;
    void* out;              // [N, heads * vdim]
    int heads, dim, vdim, partitions, stride_rows;     // stride_rows: floats from one partition's staged rows to the next's
    float eps;
    // wkv: the row that the next step's token shift reads
    const void* h;
    float* shift_state;     // [slots, width]
    int width;
    // segmented form
    int segment, max_segments;  // tokens per segment, segments the scratch has room for per sequence
    int groups;                 // delta, pass A: blocks per (segment, head): one for the value columns + those for the transition's
    float* segment_state;       // [S, max_segments, heads, dim, vdim]: pass A leaves L there, the scan S_in
    float* segment_move;        // wkv: [S, max_segments, heads, dim], the products of the decays; delta: [.., heads, dim, dim]
};

enum : int { REC_WKV = 0, REC_DELTA = 1 };
// PASS 0: a sequence's tokens in one pass, from and into its state slot.  1: pass A of the segmented form.  3: pass C.
enum : int { REC_ONE_PASS = 0, REC_LOCAL = 1, REC_OUTPUT = 3 };

template <typename T, typename W, int R, int MODE, int PASS>
__global__ void __launch_bounds__(512, R <= 8 ? 2 : 1) matrix_recurrence_kernel(RecArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float4 rec_shared_raw[];
    float* shared = reinterpret_cast<float*>(rec_shared_raw);
    const int seq = blockIdx.x, head = blockIdx.y;
    int begin = a.q_start[seq], end = a.q_start[seq + 1];
    if (begin >= end) return;
    const int seq_end = end;
    bool last_segment = true;
    size_t segment_index = 0;
    int group = 0;      // delta, pass A: 0: the value columns; g > 0: columns (g - 1) vdim ... of the transition
    if (PASS != REC_ONE_PASS) {
        const int segments = (end - begin + a.segment - 1) / a.segment;
        const int groups = (PASS == REC_LOCAL && MODE == REC_DELTA) ? a.groups : 1;
        const int segment = blockIdx.z / groups;
        group = blockIdx.z % groups;
        if (segment >= segments) return;
        last_segment = segment == segments - 1;
        if (PASS == REC_LOCAL && last_segment) return;      // nobody needs what a zero start leaves behind the last one
        begin += segment * a.segment;
        end = min(end, begin + a.segment);
        segment_index = ((size_t)seq * a.max_segments + segment) * a.heads + head;
    }
    const int dim = a.dim, vdim = a.vdim, P = a.partitions, padded = P * a.stride_rows;
    float* q_s = shared;                               // [REC_TOKENS][padded]   wkv: r
    float* k_s = q_s + REC_TOKENS * padded;
    float* w_s = k_s + REC_TOKENS * padded;            // wkv only: the decays
    float* v_s = w_s + (MODE == REC_WKV ? REC_TOKENS * padded : 0);     // [REC_TOKENS][vdim]
    float* o_s = v_s + REC_TOKENS * vdim;              // [REC_TOKENS][vdim]
    float* scalar_s = o_s + REC_TOKENS * vdim;         // [REC_TOKENS][2]: wkv: the bonus term; delta: g and beta
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int per_warp = 32 / P;                       // columns of S per warp
    const int part = lane / per_warp, column = warp * per_warp + lane % per_warp;
    const int row0 = part * R;
    const int move_column = (group - 1) * vdim + column;      // this thread's column of the transition (group > 0)
    const bool owner = column < vdim && (group == 0 || move_column < dim);
    const T* proj = (const T*)a.proj;
    const int slot = a.state_slots[seq];

    float S[R];
    float decay[(PASS == REC_LOCAL && MODE == REC_WKV) ? R : 1];      // pass A: the product of the segment's decays, row by row
    float* state = a.state + ((size_t)slot * a.heads + head) * dim * vdim;
    float* segment_state = a.segment_state + segment_index * dim * vdim;
    const float* source = PASS == REC_OUTPUT ? segment_state : state;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        if (PASS == REC_LOCAL) S[i] = (group > 0 && row0 + i == move_column) ? 1.0f : 0.0f;
        else S[i] = (owner && row0 + i < dim) ? source[(size_t)(row0 + i) * vdim + column] : 0.0f;
        if (PASS == REC_LOCAL && MODE == REC_WKV) decay[i] = 1.0f;
    }

    const int qk_head = MODE == REC_DELTA ? head / (a.heads / a.qk_heads) : head;
    for (int first = begin; first < end; first += REC_TOKENS) {
        const int count = min(REC_TOKENS, end - first);
        __syncthreads();      // the staged values of the tokens before have been read
        // ---- stage: a warp per token
        for (int t = warp; t < count; t += warps) {
            const size_t token = (size_t)(first + t);
            float bonus = 0.0f;
            for (int i = lane; i < P * R; i += 32) {
                float qv = 0.0f, kv = 0.0f, wv = 0.0f;
                if (i < dim) {
                    if (MODE == REC_WKV) {
                        const T* row = proj + token * a.row_width;
                        kv = Num<T>::load(row + a.k_offset + head * dim + i);
                        wv = expf(-expf(a.wide[token * a.heads * dim + head * dim + i] + a.w0[head * dim + i]));
                        if (PASS != REC_LOCAL) {
                            qv = Num<T>::load(row + a.r_offset + head * dim + i);
                            bonus = fmaf(qv * a.bonus[head * dim + i], kv, bonus);
                        }
                    } else {
                        if (PASS != REC_LOCAL) qv = a.pre[token * a.pre_width + a.q_col + qk_head * dim + i];
                        kv = a.pre[token * a.pre_width + a.k_col + qk_head * dim + i];
                    }
                }
                const int at = t * padded + (i / R) * a.stride_rows + i % R;
                q_s[at] = qv;
                k_s[at] = kv;
                if (MODE == REC_WKV) w_s[at] = wv;
            }
            for (int j = lane; j < vdim; j += 32)
                v_s[t * vdim + j] = group > 0 ? 0.0f
                                    : MODE == REC_WKV ? Num<T>::load(proj + token * a.row_width + a.v_offset + head * vdim + j)
                                                      : a.pre[token * a.pre_width + a.v_col + head * vdim + j];
            if (MODE == REC_WKV) {
                bonus = warp_sum(bonus);
                if (lane == 0) scalar_s[2 * t] = bonus;
            } else if (lane == 0) {
                const float b = a.wide[token * 2 * a.heads + head], z = a.wide[token * 2 * a.heads + a.heads + head] + a.dt_bias[head];
                const float softplus = z > 20.0f ? z : log1pf(expf(z));
                scalar_s[2 * t] = expf(-expf(a.a_log[head]) * softplus);
                scalar_s[2 * t + 1] = 1.0f / (1.0f + expf(-b));
            }
        }
        __syncthreads();
        // ---- walk the tokens on the registers
        for (int t = 0; t < count; ++t) {
            const float vj = owner ? v_s[t * vdim + column] : 0.0f;
            const float4* q4 = reinterpret_cast<const float4*>(q_s + t * padded + part * a.stride_rows);
            const float4* k4 = reinterpret_cast<const float4*>(k_s + t * padded + part * a.stride_rows);
            float o;
            if (MODE == REC_WKV) {
                const float4* w4 = reinterpret_cast<const float4*>(w_s + t * padded + part * a.stride_rows);
                if (PASS == REC_LOCAL) {
#pragma unroll
                    for (int i = 0; i < R / 4; ++i) {
                        const float4 kk = k4[i], ww = w4[i];
                        S[4 * i + 0] = fmaf(ww.x, S[4 * i + 0], kk.x * vj);
                        S[4 * i + 1] = fmaf(ww.y, S[4 * i + 1], kk.y * vj);
                        S[4 * i + 2] = fmaf(ww.z, S[4 * i + 2], kk.z * vj);
                        S[4 * i + 3] = fmaf(ww.w, S[4 * i + 3], kk.w * vj);
                        decay[(4 * i + 0) % (sizeof(decay) / sizeof(float))] *= ww.x;
                        decay[(4 * i + 1) % (sizeof(decay) / sizeof(float))] *= ww.y;
                        decay[(4 * i + 2) % (sizeof(decay) / sizeof(float))] *= ww.z;
                        decay[(4 * i + 3) % (sizeof(decay) / sizeof(float))] *= ww.w;
                    }
                    continue;
                }
                float sum = 0.0f;
#pragma unroll
                for (int i = 0; i < R / 4; ++i) {
                    const float4 rr = q4[i], kk = k4[i], ww = w4[i];
                    sum = fmaf(rr.x, S[4 * i + 0], sum);
                    sum = fmaf(rr.y, S[4 * i + 1], sum);
                    sum = fmaf(rr.z, S[4 * i + 2], sum);
                    sum = fmaf(rr.w, S[4 * i + 3], sum);
                    S[4 * i + 0] = fmaf(ww.x, S[4 * i + 0], kk.x * vj);
                    S[4 * i + 1] = fmaf(ww.y, S[4 * i + 1], kk.y * vj);
                    S[4 * i + 2] = fmaf(ww.z, S[4 * i + 2], kk.z * vj);
                    S[4 * i + 3] = fmaf(ww.w, S[4 * i + 3], kk.w * vj);
                }
                for (int offset = per_warp; offset < 32; offset <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
                o = fmaf(scalar_s[2 * t], vj, sum);
            } else {
                const float g = scalar_s[2 * t], beta = scalar_s[2 * t + 1];
                float read = 0.0f;
#pragma unroll
                for (int i = 0; i < R / 4; ++i) {
                    const float4 kk = k4[i];
                    read = fmaf(S[4 * i + 0], kk.x, read);
                    read = fmaf(S[4 * i + 1], kk.y, read);
                    read = fmaf(S[4 * i + 2], kk.z, read);
                    read = fmaf(S[4 * i + 3], kk.w, read);
                }
                for (int offset = per_warp; offset < 32; offset <<= 1) read += __shfl_xor_sync(0xffffffffu, read, offset);
                const float d = beta * (vj - g * read);
                asm volatile("" ::: "memory");      // the keys are read again below rather than held in registers meanwhile
                if (PASS == REC_LOCAL) {
#pragma unroll
                    for (int i = 0; i < R / 4; ++i) {
                        const float4 kk = k4[i];
                        S[4 * i + 0] = fmaf(g, S[4 * i + 0], kk.x * d);
                        S[4 * i + 1] = fmaf(g, S[4 * i + 1], kk.y * d);
                        S[4 * i + 2] = fmaf(g, S[4 * i + 2], kk.z * d);
                        S[4 * i + 3] = fmaf(g, S[4 * i + 3], kk.w * d);
                    }
                    continue;
                }
                float sum = 0.0f;
#pragma unroll
                for (int i = 0; i < R / 4; ++i) {
                    const float4 qq = q4[i], kk = k4[i];
                    S[4 * i + 0] = fmaf(g, S[4 * i + 0], kk.x * d);
                    S[4 * i + 1] = fmaf(g, S[4 * i + 1], kk.y * d);
                    S[4 * i + 2] = fmaf(g, S[4 * i + 2], kk.z * d);
                    S[4 * i + 3] = fmaf(g, S[4 * i + 3], kk.w * d);
                    sum = fmaf(S[4 * i + 0], qq.x, sum);
                    sum = fmaf(S[4 * i + 1], qq.y, sum);
                    sum = fmaf(S[4 * i + 2], qq.z, sum);
                    sum = fmaf(S[4 * i + 3], qq.w, sum);
                }
                for (int offset = per_warp; offset < 32; offset <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
                o = sum;
            }
            if (owner && part == 0) o_s[t * vdim + column] = o;
        }
        if (PASS == REC_LOCAL) continue;
        __syncthreads();
        // ---- head norm, gate, store: a warp per token
        for (int t = warp; t < count; t += warps) {
            float squares = 0.0f;
            for (int j = lane; j < vdim; j += 32) squares = fmaf(o_s[t * vdim + j], o_s[t * vdim + j], squares);
            const float inverse = rsqrtf(warp_sum(squares) / (float)vdim + a.eps);
            const T* g_row = proj + (size_t)(first + t) * a.row_width + a.g_offset + head * vdim;
            T* dst = (T*)a.out + ((size_t)(first + t) * a.heads + head) * vdim;
            const W* weight = (const W*)a.weight + (size_t)head * a.weight_stride;
            for (int j = lane; j < vdim; j += 32) {
                const float g = Num<T>::load(g_row + j);
                Num<T>::store(dst + j, o_s[t * vdim + j] * inverse * Num<W>::load(weight + j) * (g / (1.0f + expf(-g))));
            }
        }
    }
    if (PASS == REC_LOCAL) {
        if (owner && group == 0) {
#pragma unroll
            for (int i = 0; i < R; ++i)
                if (row0 + i < dim) segment_state[(size_t)(row0 + i) * vdim + column] = S[i];
        }
        if (MODE == REC_DELTA && owner && group > 0) {
            float* move = a.segment_move + segment_index * dim * dim;
#pragma unroll
            for (int i = 0; i < R; ++i)
                if (row0 + i < dim) move[(size_t)(row0 + i) * dim + move_column] = S[i];
        }
        if (MODE == REC_WKV && column == 0) {
#pragma unroll
            for (int i = 0; i < R; ++i)
                if (row0 + i < dim) a.segment_move[segment_index * dim + row0 + i] = decay[i % (sizeof(decay) / sizeof(float))];
        }
        return;
    }
    if (!last_segment) return;
    if (owner) {
#pragma unroll
        for (int i = 0; i < R; ++i)
            if (row0 + i < dim) state[(size_t)(row0 + i) * vdim + column] = S[i];
    }
    if (MODE == REC_WKV && a.shift_state) {
        // the sequence's last row of this step is what its next token mixes with; the heads share the copy
        const T* last = (const T*)a.h + (size_t)(seq_end - 1) * a.width;
        for (int c = head * blockDim.x + threadIdx.x; c < a.width; c += a.heads * blockDim.x)
            a.shift_state[(size_t)slot * a.width + c] = Num<T>::load(last + c);
    }
}

// The scan between the passes, per (sequence, head): S_in(0) is the slot's state and S_in(k + 1) = M_k S_in(k) + L_k; S_in(k)
// takes L_k's place in the scratch.  With a diagonal M (wkv) the cells are independent: one thread per cell, the
// segments' values loaded a few ahead of the chain of multiply-adds that needs them.
__global__ void rec_scan_diagonal_kernel(RecArgs a) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int tokens = a.q_start[seq + 1] - a.q_start[seq];
    if (tokens <= 0) return;
    const int segments = (tokens + a.segment - 1) / a.segment;
    const int cells = a.dim * a.vdim;
    const int cell = blockIdx.z * blockDim.x + threadIdx.x;
    if (cell >= cells) return;
    const int row = cell / a.vdim;
    float S = a.state[((size_t)a.state_slots[seq] * a.heads + head) * cells + cell];
    const size_t first = ((size_t)seq * a.max_segments) * a.heads + head;
    const size_t stride = a.heads;      // from one segment's index to the next's
    constexpr int AHEAD = 4;
    for (int k0 = 0; k0 < segments; k0 += AHEAD) {
        float local[AHEAD], decay[AHEAD];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            const int k = k0 + u;
            const bool more = k + 1 < segments;
            const size_t index = first + (size_t)k * stride;
            local[u] = more ? a.segment_state[index * cells + cell] : 0.0f;
            decay[u] = more ? a.segment_move[index * a.dim + row] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            const int k = k0 + u;
            if (k < segments) {
                a.segment_state[(first + (size_t)k * stride) * cells + cell] = S;
                if (k + 1 < segments) S = fmaf(decay[u], S, local[u]);
            }
        }
    }
}

// With a full M (the delta rule) a column of S_in(k + 1) needs the whole column of S_in(k): a block keeps `chunk` columns
// of the running state in shared memory, a thread up to SCAN_CELLS cells of them, each a sum over dim in a fixed order.
#define SCAN_CELLS 8
#define SCAN_THREADS 256
__global__ void __launch_bounds__(SCAN_THREADS) rec_scan_matrix_kernel(RecArgs a, int chunk) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float4 scan_shared_raw[];
    float* running = reinterpret_cast<float*>(scan_shared_raw);      // [dim][chunk]
    const int seq = blockIdx.x, head = blockIdx.y, column0 = blockIdx.z * chunk;
    const int tokens = a.q_start[seq + 1] - a.q_start[seq];
    if (tokens <= 0) return;
    const int segments = (tokens + a.segment - 1) / a.segment;
    const int dim = a.dim, vdim = a.vdim;
    const int columns = min(chunk, vdim - column0);
    const float* state = a.state + ((size_t)a.state_slots[seq] * a.heads + head) * dim * vdim;
    const size_t first = ((size_t)seq * a.max_segments) * a.heads + head;
    float S[SCAN_CELLS], local[SCAN_CELLS];
    int row[SCAN_CELLS], col[SCAN_CELLS];
    bool valid[SCAN_CELLS];
#pragma unroll
    for (int u = 0; u < SCAN_CELLS; ++u) {
        const int e = threadIdx.x + u * SCAN_THREADS;
        row[u] = e / chunk;
        col[u] = e % chunk;
        valid[u] = row[u] < dim && col[u] < columns;
        S[u] = valid[u] ? state[(size_t)row[u] * vdim + column0 + col[u]] : 0.0f;
    }
    for (int k = 0; k < segments; ++k) {
        const size_t index = first + (size_t)k * a.heads;
        float* segment_state = a.segment_state + index * dim * vdim;
        const float* move = a.segment_move + index * dim * dim;
        const bool more = k + 1 < segments;
        __syncthreads();      // the running state of the segment before has been read
#pragma unroll
        for (int u = 0; u < SCAN_CELLS; ++u) {
            if (!valid[u]) continue;
            float* cell = segment_state + (size_t)row[u] * vdim + column0 + col[u];
            local[u] = more ? *cell : 0.0f;
            *cell = S[u];
            running[row[u] * chunk + col[u]] = S[u];
        }
        __syncthreads();
        if (!more) break;
#pragma unroll
        for (int u = 0; u < SCAN_CELLS; ++u) {
            if (!valid[u]) continue;
            const float* m_row = move + (size_t)row[u] * dim;
            float part[4] = {local[u], 0.0f, 0.0f, 0.0f};
            int m = 0;
            for (; m + 4 <= dim; m += 4) {
                part[0] = fmaf(m_row[m + 0], running[(m + 0) * chunk + col[u]], part[0]);
                part[1] = fmaf(m_row[m + 1], running[(m + 1) * chunk + col[u]], part[1]);
                part[2] = fmaf(m_row[m + 2], running[(m + 2) * chunk + col[u]], part[2]);
                part[3] = fmaf(m_row[m + 3], running[(m + 3) * chunk + col[u]], part[3]);
            }
            for (; m < dim; ++m) part[0] = fmaf(m_row[m], running[m * chunk + col[u]], part[0]);
            S[u] = (part[0] + part[1]) + (part[2] + part[3]);
        }
    }
}

// The same scan for heads of up to SCAN_STAGED_DIM key channels (a multiple of four): the transition of the next segment
// is copied into shared memory (cp.async, two buffers) while this segment's product runs from shared memory, a thread
// one row of 4 * C4 columns.  The sum over the key channels runs in ascending order.
#define SCAN_STAGED_DIM 128
template <int C4>
__global__ void __launch_bounds__(2 * SCAN_STAGED_DIM) rec_scan_matrix_staged_kernel(RecArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float4 scan_shared_raw[];
    constexpr int CHUNK = 8 * C4;          // columns per block: two threads per row, 4 * C4 columns each
    const int dim = a.dim, vdim = a.vdim, stride = dim + 4;
    float* move_s = reinterpret_cast<float*>(scan_shared_raw);      // [2][dim][stride]
    float* running = move_s + 2 * dim * stride;                     // [dim][CHUNK]
    const int seq = blockIdx.x, head = blockIdx.y, column0 = blockIdx.z * CHUNK;
    const int tokens = a.q_start[seq + 1] - a.q_start[seq];
    if (tokens <= 0) return;
    const int segments = (tokens + a.segment - 1) / a.segment;
    const size_t first = ((size_t)seq * a.max_segments) * a.heads + head;
    const int row = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * (4 * C4);
    const bool row_valid = row < dim;
    const float* state = a.state + ((size_t)a.state_slots[seq] * a.heads + head) * dim * vdim;
    float S[4 * C4], local[4 * C4];
#pragma unroll
    for (int j = 0; j < 4 * C4; ++j) {
        const int column = column0 + c0 + j;
        S[j] = (row_valid && column < vdim) ? state[(size_t)row * vdim + column] : 0.0f;
    }
    const int quads = dim * dim / 4;      // 16-byte pieces of a transition
    auto fetch = [&](int k) {
        const float* move = a.segment_move + (first + (size_t)k * a.heads) * dim * dim;
        float* dst = move_s + (k & 1) * dim * stride;
        for (int f = threadIdx.x; f < quads; f += blockDim.x) {
            const int r = f / (dim / 4), c = (f % (dim / 4)) * 4;
            const unsigned target = (unsigned)__cvta_generic_to_shared(dst + r * stride + c);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(target), "l"(move + (size_t)r * dim + c) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // what segment k leaves from a zero state (nothing behind the last one); read a segment ahead of its use
    auto read_local = [&](int k, float* into) {
        const float* segment_state = a.segment_state + (first + (size_t)k * a.heads) * dim * vdim;
#pragma unroll
        for (int j = 0; j < 4 * C4; ++j) {
            const int column = column0 + c0 + j;
            into[j] = (k + 1 < segments && row_valid && column < vdim) ? segment_state[(size_t)row * vdim + column] : 0.0f;
        }
    };
    float next_local[4 * C4];
    if (segments > 1) fetch(0);
    read_local(0, next_local);
    for (int k = 0; k < segments; ++k) {
        const bool more = k + 1 < segments, ahead = k + 2 < segments;
        if (ahead) fetch(k + 1);
        float* segment_state = a.segment_state + (first + (size_t)k * a.heads) * dim * vdim;
#pragma unroll
        for (int j = 0; j < 4 * C4; ++j) {
            const int column = column0 + c0 + j;
            local[j] = next_local[j];
            if (row_valid && column < vdim) segment_state[(size_t)row * vdim + column] = S[j];
        }
        if (!more) break;
        read_local(k + 1, next_local);
        if (row_valid) {
#pragma unroll
            for (int c = 0; c < C4; ++c)
                reinterpret_cast<float4*>(running + row * CHUNK + c0)[c] = make_float4(S[4 * c], S[4 * c + 1], S[4 * c + 2], S[4 * c + 3]);
        }
        if (ahead) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();      // this segment's transition and the running state are in shared memory
        if (row_valid) {
            const float* m_row = move_s + (k & 1) * dim * stride + row * stride;
#pragma unroll
            for (int j = 0; j < 4 * C4; ++j) S[j] = local[j];
            for (int m = 0; m < dim; m += 4) {
                const float4 mm = *reinterpret_cast<const float4*>(m_row + m);
                const float factor[4] = {mm.x, mm.y, mm.z, mm.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int c = 0; c < C4; ++c) {
                        const float4 r = reinterpret_cast<const float4*>(running + (m + i) * CHUNK + c0)[c];
                        S[4 * c + 0] = fmaf(factor[i], r.x, S[4 * c + 0]);
                        S[4 * c + 1] = fmaf(factor[i], r.y, S[4 * c + 1]);
                        S[4 * c + 2] = fmaf(factor[i], r.z, S[4 * c + 2]);
                        S[4 * c + 3] = fmaf(factor[i], r.w, S[4 * c + 3]);
                    }
                }
            }
        }
        __syncthreads();      // the running state and this buffer have been read
    }
}

// Rows of S per thread and row partitions per warp (a power of two) for heads of `dim` x `vdim`: the fewest rows with
// which a block has at most 512 threads; 0: no arrangement (64 rows per thread already spill some).
static int rec_rows_per_thread(int dim, int vdim, int* partitions) {
    const int choices[4] = {8, 16, 32, 64};
    for (int c = 0; c < 4; ++c) {
        int parts = 1;
        while (parts * choices[c] < dim) parts *= 2;
        if (parts > 32) continue;
        const int per_warp = 32 / parts;
        if ((vdim + per_warp - 1) / per_warp * 32 <= 512) {
            *partitions = parts;
            return choices[c];
        }
    }
    return 0;
}

LLM_EXPORT int llm_matrix_recurrence_supports(int dim, int vdim) {
    int partitions;
    return dim > 0 && vdim > 0 && rec_rows_per_thread(dim, vdim, &partitions) != 0;
}

// The staged scan: 8 columns per block; 16 where blocks of 8 would be more than one per SM (its shared memory allows one).
static int rec_launch_staged_scan(RecArgs& a, int n_seqs, cudaStream_t stream) {
    const bool wide = (size_t)n_seqs * a.heads * ((a.vdim + 7) / 8) > 148;
    const int chunk = wide ? 16 : 8;
    const size_t shared = ((size_t)2 * a.dim * (a.dim + 4) + (size_t)a.dim * chunk) * sizeof(float);
    const void* kernel = wide ? (const void*)rec_scan_matrix_staged_kernel<2> : (const void*)rec_scan_matrix_staged_kernel<1>;
    if (shared > 40 * 1024) {
        const int status = llm_raise_shared_limit(kernel, shared, "matrix recurrence scan");
        if (status != LLM_OK) return status;
    }
    const dim3 grid(n_seqs, a.heads, (a.vdim + chunk - 1) / chunk);
    if (wide) llm_launch(rec_scan_matrix_staged_kernel<2>, grid, 2 * SCAN_STAGED_DIM, shared, stream, a);
    else llm_launch(rec_scan_matrix_staged_kernel<1>, grid, 2 * SCAN_STAGED_DIM, shared, stream, a);
    return LLM_OK;
}

static int rec_launch(RecArgs& a, int mode, int n_seqs, int dtype, int weight_dtype, cudaStream_t stream) {
    if (n_seqs == 0) return LLM_OK;
    const bool segmented = a.segment > 0;
    if (segmented && (a.max_segments <= 0 || !a.segment_state || !a.segment_move)) {
        llm_set_error("matrix recurrence: the segmented form needs its scratch");
        return LLM_REFUSED;
    }
    int partitions = 0;
    const int rows = a.heads > 0 ? rec_rows_per_thread(a.dim, a.vdim, &partitions) : 0;
    if (!rows) {
        llm_set_error("matrix recurrence: %d heads of %d key and %d value channels are not supported", a.heads, a.dim, a.vdim);
        return LLM_REFUSED;
    }
    a.partitions = partitions;
    a.stride_rows = rows + 4;       // four floats between the partitions' rows: their 16-byte reads fall into different banks
    const int per_warp = 32 / partitions;
    const int threads = (a.vdim + per_warp - 1) / per_warp * 32;
    const int padded = partitions * a.stride_rows;
    const size_t shared = ((size_t)(mode == REC_WKV ? 3 : 2) * REC_TOKENS * padded + (size_t)2 * REC_TOKENS * a.vdim + 2 * REC_TOKENS) * sizeof(float);
    a.groups = 1 + (a.dim + a.vdim - 1) / a.vdim;
    // the scan of the delta rule: columns per block such that a thread has at most SCAN_CELLS cells
    int chunk = SCAN_CELLS * SCAN_THREADS / a.dim;
    if (chunk > 8) chunk = 8;
    if (chunk > a.vdim) chunk = a.vdim;
    const bool staged_scan = a.dim <= SCAN_STAGED_DIM && a.dim % 4 == 0;
    if (segmented && mode == REC_DELTA && chunk < 1) {
        llm_set_error("matrix recurrence: the segmented delta rule takes heads of up to %d key channels", SCAN_CELLS * SCAN_THREADS);
        return LLM_REFUSED;
    }
#define REC_LAUNCH_PASS(R, MODE, PASS, GRID)                                                                               \
    do {                                                                                                                   \
        if (shared > 40 * 1024) {                                                                                          \
            const int status = llm_raise_shared_limit((const void*)matrix_recurrence_kernel<T, W, R, MODE, PASS>, shared, "matrix recurrence"); \
            if (status != LLM_OK) return status;                                                                           \
        }                                                                                                                  \
        llm_launch(matrix_recurrence_kernel<T, W, R, MODE, PASS>, GRID, threads, shared, stream, a);                       \
    } while (0)
#define REC_LAUNCH(R, MODE)                                                                                                \
    do {                                                                                                                   \
        if (!segmented) {                                                                                                  \
            REC_LAUNCH_PASS(R, MODE, REC_ONE_PASS, dim3(n_seqs, a.heads));                                                 \
        } else {                                                                                                           \
            REC_LAUNCH_PASS(R, MODE, REC_LOCAL, dim3(n_seqs, a.heads, a.max_segments * (MODE == REC_DELTA ? a.groups : 1))); \
            if (MODE == REC_WKV)                                                                                           \
                llm_launch(rec_scan_diagonal_kernel, dim3(n_seqs, a.heads, (a.dim * a.vdim + 255) / 256), 256, 0, stream, a); \
            else if (staged_scan) {                                                                                        \
                const int status = rec_launch_staged_scan(a, n_seqs, stream);                                              \
                if (status != LLM_OK) return status;                                                                       \
            } else                                                                                                         \
                llm_launch(rec_scan_matrix_kernel, dim3(n_seqs, a.heads, (a.vdim + chunk - 1) / chunk), SCAN_THREADS,      \
                           (size_t)a.dim * chunk * sizeof(float), stream, a, chunk);                                       \
            REC_LAUNCH_PASS(R, MODE, REC_OUTPUT, dim3(n_seqs, a.heads, a.max_segments));                                   \
        }                                                                                                                  \
    } while (0)
#define REC_LAUNCH_ROWS(MODE)                                                                                              \
    do {                                                                                                                   \
        if (rows == 8) REC_LAUNCH(8, MODE);                                                                                \
        else if (rows == 16) REC_LAUNCH(16, MODE);                                                                         \
        else if (rows == 32) REC_LAUNCH(32, MODE);                                                                         \
        else REC_LAUNCH(64, MODE);                                                                                         \
    } while (0)
    LLM_DISPATCH_DTYPE_WEIGHT(dtype, weight_dtype, {
        if (mode == REC_WKV) REC_LAUNCH_ROWS(REC_WKV);
        else REC_LAUNCH_ROWS(REC_DELTA);
    });
#undef REC_LAUNCH_ROWS
#undef REC_LAUNCH
#undef REC_LAUNCH_PASS
    return llm_check_launch("matrix recurrence");
}

LLM_EXPORT int llm_wkv_recurrent(const void* proj, int row_width, int r_offset, int k_offset, int v_offset, int g_offset,
                                 const float* z, const float* w0, const float* bonus, const void* weight, float* state,
                                 const int* state_slots, const int* q_start, void* out, int n_seqs, int heads, int dim, float eps,
                                 const void* h, float* shift_state, int width, int dtype, int weight_dtype, int segment, int max_segments,
                                 float* segment_state, float* segment_move, cudaStream_t stream) {
    RecArgs a = {};
    a.segment = segment; a.max_segments = max_segments; a.segment_state = segment_state; a.segment_move = segment_move;
    a.proj = proj; a.row_width = row_width; a.r_offset = r_offset; a.k_offset = k_offset; a.v_offset = v_offset; a.g_offset = g_offset;
    a.wide = z; a.w0 = w0; a.bonus = bonus; a.weight = weight; a.weight_stride = dim; a.state = state; a.state_slots = state_slots;
    a.q_start = q_start; a.out = out; a.heads = heads; a.dim = dim; a.vdim = dim; a.eps = eps; a.h = h; a.shift_state = shift_state;
    a.width = width; a.qk_heads = heads;
    return rec_launch(a, REC_WKV, n_seqs, dtype, weight_dtype, stream);
}

LLM_EXPORT int llm_delta_rule_recurrent(const void* proj, int row_width, int g_offset, const float* pre, int pre_width, int q_col,
                                        int k_col, int v_col, const float* wide, const float* a_log, const float* dt_bias,
                                        const void* weight, float* state, const int* state_slots, const int* q_start, void* out,
                                        int n_seqs, int heads, int qk_heads, int dim, int vdim, float eps, int dtype, int weight_dtype,
                                        int segment, int max_segments, float* segment_state, float* segment_move,
                                        cudaStream_t stream) {
    if (qk_heads <= 0 || heads % qk_heads) {
        llm_set_error("delta_rule_recurrent: %d heads are no multiple of %d query/key heads", heads, qk_heads);
        return LLM_REFUSED;
    }
    RecArgs a = {};
    a.proj = proj; a.row_width = row_width; a.g_offset = g_offset; a.pre = pre; a.pre_width = pre_width; a.q_col = q_col;
    a.k_col = k_col; a.v_col = v_col; a.qk_heads = qk_heads; a.wide = wide; a.a_log = a_log; a.dt_bias = dt_bias; a.weight = weight;
    a.segment = segment; a.max_segments = max_segments; a.segment_state = segment_state; a.segment_move = segment_move;
    a.weight_stride = 0; a.state = state; a.state_slots = state_slots; a.q_start = q_start; a.out = out; a.heads = heads;
    a.dim = dim; a.vdim = vdim; a.eps = eps;
    return rec_launch(a, REC_DELTA, n_seqs, dtype, weight_dtype, stream);
}
