// What stands around the mixers of layers that keep several residual streams, shift their input by a token, run two
// mixers side by side, or attend over a shared latent instead of per-head keys and values.
//
// Residual streams (hyper-connections): instead of one residual row a token has S of them, [tokens, S, width] fp32.
// A sublayer reads u = sum_s in[s] x_s through its norm, and its result y goes back as
//   x_r <- sum_s mix[s, r] x_s + out[r] y      for all r at once, from the old streams.
// `streams_step` does the write of one sublayer and the read (with the RMS norm) of the next in one pass over the
// token's streams; either half may be left out.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

struct StreamWeights {
    float mix[MAX_STREAMS * MAX_STREAMS];  // [from, to]
    float out[MAX_STREAMS];
    float in[MAX_STREAMS];
};

__global__ void __launch_bounds__(256) streams_expand_kernel(const float* h, float* __restrict__ xs, int streams, int width) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = h[(size_t)t * width + c];
        for (int s = 0; s < streams; ++s) xs[((size_t)t * streams + s) * width + c] = v;
    }
}

__global__ void __launch_bounds__(256) streams_sum_kernel(const float* xs, float* __restrict__ h, int streams, int width) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = 0.0f;
        for (int s = 0; s < streams; ++s) v += xs[((size_t)t * streams + s) * width + c];
        h[(size_t)t * width + c] = v;
    }
}

// write (y not null): the streams take the sublayer's result; read (norm_w not null): out = rmsnorm(sum_s in[s] x_s) * norm_w.
// mix, out_w, in_w lie in device memory (learned tensors), fp32.
template <typename T>
__global__ void __launch_bounds__(512) streams_step_kernel(float* xs, const float* y, const float* __restrict__ mix,
                                                           const float* __restrict__ out_w, const float* __restrict__ in_w,
                                                           const float* __restrict__ norm_w, float eps, T* __restrict__ out,
                                                           int streams, int width, const float* __restrict__ shift,
                                                           float* shift_state, const int* __restrict__ positions,
                                                           const int* __restrict__ seq_state_slot) {
    extern __shared__ float u_row[];  // [width], the read's sum (only with a read)
    __shared__ float scratch[33];
    __shared__ StreamWeights sw;
    const bool writes = y != nullptr, reads = norm_w != nullptr;
    // the learned numbers are weights: they may be read before the launch before this one has ended
    if (threadIdx.x < streams * streams && writes) sw.mix[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < streams) {
        if (writes) sw.out[threadIdx.x] = out_w[threadIdx.x];
        if (reads) sw.in[threadIdx.x] = in_w[threadIdx.x];
    }
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    float* row = xs + (size_t)t * streams * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float x[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) x[s] = s < streams ? row[(size_t)s * width + c] : 0.0f;
        if (writes) {
            const float yy = y[(size_t)t * width + c];
            float nx[MAX_STREAMS];
#pragma unroll
            for (int r = 0; r < MAX_STREAMS; ++r) {
                float a = 0.0f;
                if (r < streams) {
#pragma unroll
                    for (int s = 0; s < MAX_STREAMS; ++s)
                        if (s < streams) a = fmaf(sw.mix[s * streams + r], x[s], a);
                    a = fmaf(sw.out[r], yy, a);
                    row[(size_t)r * width + c] = a;
                }
                nx[r] = a;
            }
#pragma unroll
            for (int r = 0; r < MAX_STREAMS; ++r) x[r] = nx[r];
        }
        if (reads) {
            float u = 0.0f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < streams) u = fmaf(sw.in[s], x[s], u);
            u_row[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!reads) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    if (!shift) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)t * width + c] = from_float<T>((u_row[c] * inv) * norm_w[c]);
        return;
    }
    // A step of single tokens (row t is request t's only token): the token shift of the normed row right here, from and
    // to the request's state, on the row as it is rounded for the mixer (what the kernels of its own do as well).
    const int pos = positions[t];
    float* st = shift_state + (size_t)seq_state_slot[t] * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float own = to_float(from_float<T>((u_row[c] * inv) * norm_w[c]));
        const float prev = pos == 0 ? 0.0f : st[c];
        st[c] = own;
        out[(size_t)t * width + c] = from_float<T>(fmaf(prev - own, shift[c], own));
    }
}

// ---------------------------------------------------------------------------------------------
// Token shift: a mixer's input row x_t becomes x_t + (x_(t-1) - x_t) * shift, with x_(t-1) the row of the token before
// as it was BEFORE its own shift (zeros for a sequence's first token).  The last unshifted row of a request is its
// state ([slots, width] fp32).  `apply` only reads the state and `advance` then writes it (a block that advanced it
// could otherwise overtake one that still reads it); a step of single tokens does both in one launch.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) token_shift_apply_kernel(const T* x, T* __restrict__ out, const float* __restrict__ shift,
                                                                float* state, const int* __restrict__ token_seq,
                                                                const int* __restrict__ positions,
                                                                const int* __restrict__ seq_start_pos,
                                                                const int* __restrict__ seq_state_slot, int width, int single) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int seq = token_seq[t];
    const int pos = positions[t];
    float* st = state + (size_t)seq_state_slot[seq] * width + c;
    const float own = to_float(x[(size_t)t * width + c]);
    float prev;
    if (pos == 0)
        prev = 0.0f;
    else if (pos == seq_start_pos[seq])
        prev = *st;
    else
        prev = to_float(x[(size_t)(t - 1) * width + c]);
    out[(size_t)t * width + c] = from_float<T>(fmaf(prev - own, shift[c], own));
    if (single) *st = own;
}

template <typename T>
__global__ void __launch_bounds__(256) token_shift_advance_kernel(const T* x, float* state, const int* __restrict__ seq_q_start,
                                                                  const int* __restrict__ seq_state_slot, int width) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int last = seq_q_start[seq + 1] - 1;
    if (last < seq_q_start[seq]) return;
    state[(size_t)seq_state_slot[seq] * width + c] = to_float(x[(size_t)last * width + c]);
}

// ---------------------------------------------------------------------------------------------
// Mixers side by side: h += coef * sum_b rmsnorm(y_b) * w_b over up to four branches' results (fp32 rows).
// ---------------------------------------------------------------------------------------------
struct Branches {
    const float* y[4];
    const float* w[4];
    int n;
};

__global__ void __launch_bounds__(256) branch_norm_sum_kernel(Branches br, float coef, float eps, float* h, int width,
                                                              int accumulate) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    float inv[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        inv[b] = 0.0f;
        if (b < br.n) {
            float ss = 0.0f;
            for (int c = threadIdx.x; c < width; c += blockDim.x) {
                const float v = br.y[b][(size_t)t * width + c];
                ss = fmaf(v, v, ss);
            }
            ss = block_sum(ss, scratch);
            inv[b] = 1.0f / sqrtf(ss / (float)width + eps);
        }
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float a = 0.0f;
#pragma unroll
        for (int b = 0; b < 4; ++b)
            if (b < br.n) a += (br.y[b][(size_t)t * width + c] * inv[b]) * br.w[b][c];
        h[(size_t)t * width + c] = accumulate ? fmaf(coef, a, h[(size_t)t * width + c]) : coef * a;
    }
}

// ---------------------------------------------------------------------------------------------
// Attention over a shared latent.  A token's projection row holds, per query head, [dim plain | rot rotated] query
// dimensions, and once [rank latent | rot rotated key] dimensions.  This kernel norms the latent (RMS norm with a
// weight), rotates the key part and the heads' rotated query parts (rotate-half over the first `rot_dims` of the
// part; angle = position * inv_freq[i], fp32), writes [latent | rotated key] as the token's one cache row and the
// rotated query parts into the attention's query rows behind the place of the absorbed plain part:
//   q_att[t, h] = [rank: left for the product of the plain query with the key up-projection | rot: rotated part].
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const T* proj, int ld, int q_off, int dkv_off,
                                                             const float* __restrict__ norm_w, float eps,
                                                             const int* __restrict__ positions,
                                                             const float* __restrict__ inv_freq, int rot_dims,
                                                             const int* __restrict__ slot_mapping, T* __restrict__ cache,
                                                             T* __restrict__ q_att, int ldqa, int heads, int dim, int rot,
                                                             int rank, int write_kv) {
    __shared__ float scratch[33];
    __shared__ float cs_tab[256], sn_tab[256];  // the token's angles, once for the key part and every head
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    const T* row = proj + (size_t)t * ld;
    const int half = rot_dims >> 1;
    for (int f = threadIdx.x; f < half; f += blockDim.x) sincosf(pos * inv_freq[f], &sn_tab[f], &cs_tab[f]);
    __syncthreads();
    // the heads' rotated query parts
    for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
        const int h = i / rot, e = i - h * rot;
        const T* src = row + q_off + (size_t)h * (dim + rot) + dim;
        float v = to_float(src[e]);
        if (e < rot_dims) {
            const int f = e < half ? e : e - half;
            const float sn = sn_tab[f], cs = cs_tab[f];
            const float other = to_float(src[e < half ? e + half : e - half]);
            v = e < half ? v * cs - other * sn : v * cs + other * sn;
        }
        q_att[(size_t)t * ldqa + (size_t)h * (rank + rot) + rank + e] = from_float<T>(v);
    }
    if (!write_kv) return;
    const T* dkv = row + dkv_off;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(dkv[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    T* dst = cache + (size_t)slot_mapping[t] * (rank + rot);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>((to_float(dkv[i]) * inv) * norm_w[i]);
    for (int e = threadIdx.x; e < rot; e += blockDim.x) {
        float v = to_float(dkv[rank + e]);
        if (e < rot_dims) {
            const int f = e < half ? e : e - half;
            const float sn = sn_tab[f], cs = cs_tab[f];
            const float other = to_float(dkv[rank + (e < half ? e + half : e - half)]);
            v = e < half ? v * cs - other * sn : v * cs + other * sn;
        }
        dst[rank + e] = from_float<T>(v);
    }
}

// ---------------------------------------------------------------------------------------------
// A small product per head: out[t, h, n] = (sum_k x[t, h, k] W[h, k, n]) * g, g = 1 or sigmoid(gate[t, h]).
// Eight tokens of a head stand in shared memory (fp32); a thread owns an output column for all eight and a quarter
// of the inputs, and reads each of its weights once, consecutive threads consecutive columns; the four quarters'
// sums are added in order.  fp32 FMAs.
// ---------------------------------------------------------------------------------------------
constexpr int HG_TOKENS = 8, HG_COLS = 64, HG_PARTS = 4, HG_THREADS = HG_COLS * HG_PARTS;

template <typename T>
__global__ void __launch_bounds__(HG_THREADS) head_gemm_kernel(const T* x, int ldx, int hsx, const T* __restrict__ w, T* __restrict__ out,
                                                               int ldo, int hso, const T* gate, int ldg, int tokens, int K,
                                                               int N) {
    extern __shared__ float xs[];  // [HG_TOKENS][K], then the parts' sums [HG_PARTS - 1][HG_TOKENS][HG_COLS]
    pdl_wait();
    pdl_launch_dependents();
    const int t0 = blockIdx.x * HG_TOKENS, h = blockIdx.y;
    const int cl = threadIdx.x % HG_COLS, part = threadIdx.x / HG_COLS;
    const int n = blockIdx.z * HG_COLS + cl;
    const int rows = tokens - t0 < HG_TOKENS ? tokens - t0 : HG_TOKENS;
    for (int i = threadIdx.x; i < HG_TOKENS * K; i += HG_THREADS) {
        const int r = i / K, k = i - r * K;
        xs[i] = r < rows ? to_float(x[(size_t)(t0 + r) * ldx + (size_t)h * hsx + k]) : 0.0f;
    }
    __syncthreads();
    // the inputs are cut into four runs, a quarter of the block each: four times as many weights are on their way
    float acc[HG_TOKENS];
#pragma unroll
    for (int r = 0; r < HG_TOKENS; ++r) acc[r] = 0.0f;
    const int per = (K + HG_PARTS - 1) / HG_PARTS;
    const int k0 = part * per, k1 = min(K, k0 + per);
    if (n < N) {
        const T* wh = w + (size_t)h * K * N + n;
#pragma unroll 8
        for (int k = k0; k < k1; ++k) {
            const float wv = to_float(wh[(size_t)k * N]);
#pragma unroll
            for (int r = 0; r < HG_TOKENS; ++r) acc[r] = fmaf(xs[r * K + k], wv, acc[r]);
        }
    }
    float* sums = xs + HG_TOKENS * K;
    if (part > 0) {
#pragma unroll
        for (int r = 0; r < HG_TOKENS; ++r) sums[((part - 1) * HG_TOKENS + r) * HG_COLS + cl] = acc[r];
    }
    __syncthreads();
    if (part > 0 || n >= N) return;
#pragma unroll
    for (int r = 0; r < HG_TOKENS; ++r) {
        if (r >= rows) break;
        float v = acc[r];
#pragma unroll
        for (int p = 0; p < HG_PARTS - 1; ++p) v += sums[(p * HG_TOKENS + r) * HG_COLS + cl];  // in the runs' order
        if (gate) v *= 1.0f / (1.0f + expf(-to_float(gate[(size_t)(t0 + r) * ldg + h])));
        out[(size_t)(t0 + r) * ldo + (size_t)h * hso + n] = from_float<T>(v);
    }
}

}  // namespace

FERRIS_API int ferris_streams_expand(const float* h, float* xs, int tokens, int streams, int width, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (streams <= 0 || width <= 0) FERRIS_REFUSE("streams: %d streams of %d", streams, width);
    ferris_launch(streams_expand_kernel, dim3(tokens), dim3(width >= 1024 ? 256 : 128), 0, (cudaStream_t)stream, h, xs, streams, width);
    FERRIS_LAUNCH_CHECK();
}

FERRIS_API int ferris_streams_sum(const float* xs, float* h, int tokens, int streams, int width, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (streams <= 0 || width <= 0) FERRIS_REFUSE("streams: %d streams of %d", streams, width);
    ferris_launch(streams_sum_kernel, dim3(tokens), dim3(width >= 1024 ? 256 : 128), 0, (cudaStream_t)stream, xs, h, streams, width);
    FERRIS_LAUNCH_CHECK();
}

// xs: fp32 [tokens, streams, width]; y (null: no write): fp32 [tokens, width] with mix [streams, streams] and out_w
// [streams]; norm_w (null: no read): fp32 [width] with in_w [streams], out: [tokens, width] of `dtype`.  shift (null: none;
// only where every request brings one token, row t being request t's): fp32 [width]; the read's rows are shifted towards
// shift_state[seq_state_slot[t]] (fp32 [slots, width]; zeros at position 0), which takes the unshifted row.
FERRIS_API int ferris_streams_step(float* xs, const float* y, const float* mix, const float* out_w, const float* in_w,
                                   const float* norm_w, float eps, void* out, int dtype, int tokens, int streams, int width,
                                   const float* shift, float* shift_state, const int* positions, const int* seq_state_slot,
                                   void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (streams <= 0 || streams > MAX_STREAMS || width <= 0) FERRIS_REFUSE("streams: %d streams (at most %d) of %d", streams, MAX_STREAMS, width);
    if (y && (!mix || !out_w)) FERRIS_REFUSE("streams: a write needs its mixing matrix and output weights");
    if (norm_w && (!in_w || !out)) FERRIS_REFUSE("streams: a read needs its input weights and an output");
    if (!y && !norm_w) return FERRIS_OK;
    if (shift && (!norm_w || !shift_state || !positions || !seq_state_slot)) FERRIS_REFUSE("streams: a token shift goes with a read, a state and the step's positions and slots");
    const size_t smem = norm_w ? (size_t)width * sizeof(float) : 0;
    cudaStream_t s = (cudaStream_t)stream;
    // A thread's columns are taken one after another (a column's stores stand between its loads and the next column's),
    // so in a step of few rows a row is spread over as many threads as it has pairs of columns, up to 512; with many
    // rows the SMs are busy anyway and blocks of 256 move more (2,048 rows of 4 x 2,048: 74 against 100 us).
    const int wide = tokens < 256 ? 512 : 256;
    const dim3 grid(tokens), block(width >= 1024 ? wide : (width >= 512 ? 256 : 128));
    if (dtype == FERRIS_F32) {
        int e_ = ferris_allow_dynamic_smem((const void*)streams_step_kernel<float>, smem);
        if (e_ != FERRIS_OK) return e_;
        ferris_launch(streams_step_kernel<float>, grid, block, smem, s, xs, y, mix, out_w, in_w, norm_w, eps, (float*)out, streams, width, shift, shift_state, positions, seq_state_slot);
    } else if (dtype == FERRIS_BF16) {
        int e_ = ferris_allow_dynamic_smem((const void*)streams_step_kernel<bf16>, smem);
        if (e_ != FERRIS_OK) return e_;
        ferris_launch(streams_step_kernel<bf16>, grid, block, smem, s, xs, y, mix, out_w, in_w, norm_w, eps, (bf16*)out, streams, width, shift, shift_state, positions, seq_state_slot);
    } else
        FERRIS_REFUSE("streams: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// x, out: [tokens, width] of `dtype` (out must not be x); shift: fp32 [width]; state: fp32 [slots, width].
FERRIS_API int ferris_token_shift(const void* x, void* out, int dtype, const float* shift, float* state,
                                  const int* token_seq, const int* positions, const int* seq_q_start,
                                  const int* seq_start_pos, const int* seq_state_slot, int tokens, int seqs, int width,
                                  int advance, int single_tokens, void* stream) {
    if (tokens <= 0 || seqs <= 0) return FERRIS_OK;
    if (width <= 0 || !state || !shift) FERRIS_REFUSE("token shift: width %d, or no state or weights", width);
    if (x == out) FERRIS_REFUSE("token shift: input and output must differ");
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    const int tiles = (width + threads - 1) / threads;
    if (tiles > 65535) FERRIS_REFUSE("token shift: %d columns are more than one launch takes", width);
    cudaStream_t s = (cudaStream_t)stream;
    const int single = (single_tokens && advance && tokens == seqs) ? 1 : 0;
    const dim3 block(threads), grid_a(tokens, tiles), grid_b(seqs, tiles);
    if (dtype == FERRIS_F32) {
        ferris_launch(token_shift_apply_kernel<float>, grid_a, block, 0, s, (const float*)x, (float*)out, shift, state, token_seq,
                      positions, seq_start_pos, seq_state_slot, width, single);
        if (advance && !single)
            ferris_launch(token_shift_advance_kernel<float>, grid_b, block, 0, s, (const float*)x, state, seq_q_start, seq_state_slot, width);
    } else if (dtype == FERRIS_BF16) {
        ferris_launch(token_shift_apply_kernel<bf16>, grid_a, block, 0, s, (const bf16*)x, (bf16*)out, shift, state, token_seq,
                      positions, seq_start_pos, seq_state_slot, width, single);
        if (advance && !single)
            ferris_launch(token_shift_advance_kernel<bf16>, grid_b, block, 0, s, (const bf16*)x, state, seq_q_start, seq_state_slot, width);
    } else
        FERRIS_REFUSE("token shift: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// h fp32 [tokens, width] += (accumulate) or = coef * sum_b rmsnorm(y_b) * w_b; y_b fp32 [tokens, width], w_b fp32 [width];
// 1..4 branches.
FERRIS_API int ferris_branch_norm_sum(const float* const* ys, const float* const* ws, int branches, float coef, float eps,
                                      float* h, int tokens, int width, int accumulate, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (branches < 1 || branches > 4 || width <= 0) FERRIS_REFUSE("branch norm: %d branches of %d", branches, width);
    Branches br = {};
    br.n = branches;
    for (int b = 0; b < branches; ++b) br.y[b] = ys[b], br.w[b] = ws[b];
    ferris_launch(branch_norm_sum_kernel, dim3(tokens), dim3(width >= 1024 ? 256 : 128), 0, (cudaStream_t)stream, br, coef, eps, h, width, accumulate);
    FERRIS_LAUNCH_CHECK();
}

// proj: [tokens, ld]; cache: [rows, rank + rot] (one kv head: a cache row per slot); q_att: [tokens, ldqa].
FERRIS_API int ferris_latent_prepare(const void* proj, int ld, int dtype, int q_off, int dkv_off, const float* norm_w,
                                     float eps, const int* positions, const float* inv_freq, int rot_dims,
                                     const int* slot_mapping, void* cache, void* q_att, int ldqa, int tokens, int heads,
                                     int dim, int rot, int rank, int write_kv, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (heads <= 0 || dim < 0 || rot < 0 || rank <= 0) FERRIS_REFUSE("latent prepare: %d heads of %d + %d over a latent of %d", heads, dim, rot, rank);
    if (rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || rot_dims > 512) FERRIS_REFUSE("latent prepare: %d of %d dimensions rotate (at most 512)", rot_dims, rot);
    if (rot_dims > 0 && !inv_freq) FERRIS_REFUSE("latent prepare: no frequencies");
    if (write_kv && (!slot_mapping || !cache || !norm_w)) FERRIS_REFUSE("latent prepare: no cache to write");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(latent_prepare_kernel<float>, dim3(tokens), dim3(128), 0, s, (const float*)proj, ld, q_off, dkv_off, norm_w, eps,
                      positions, inv_freq, rot_dims, slot_mapping, (float*)cache, (float*)q_att, ldqa, heads, dim, rot, rank, write_kv);
    else if (dtype == FERRIS_BF16)
        ferris_launch(latent_prepare_kernel<bf16>, dim3(tokens), dim3(128), 0, s, (const bf16*)proj, ld, q_off, dkv_off, norm_w, eps,
                      positions, inv_freq, rot_dims, slot_mapping, (bf16*)cache, (bf16*)q_att, ldqa, heads, dim, rot, rank, write_kv);
    else
        FERRIS_REFUSE("latent prepare: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// x: [tokens, ...] with head h's K inputs at column h * hsx of rows ldx apart; w: [heads, K, N]; out likewise with hso,
// ldo; gate (may be null): [tokens, ...] rows ldg apart, one number per head.
FERRIS_API int ferris_head_gemm(const void* x, int ldx, int hsx, const void* w, void* out, int ldo, int hso,
                                const void* gate, int ldg, int dtype, int tokens, int heads, int K, int N, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (heads <= 0 || heads > 65535 || K <= 0 || N <= 0) FERRIS_REFUSE("head gemm: %d heads of %d x %d", heads, K, N);
    const size_t smem = ((size_t)HG_TOKENS * K + (size_t)(HG_PARTS - 1) * HG_TOKENS * HG_COLS) * sizeof(float);
    if (smem > 200 * 1024) FERRIS_REFUSE("head gemm: %d inputs a head are more than shared memory holds", K);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((tokens + HG_TOKENS - 1) / HG_TOKENS, heads, (N + HG_COLS - 1) / HG_COLS), block(HG_THREADS);
    if (dtype == FERRIS_F32) {
        int e_ = ferris_allow_dynamic_smem((const void*)head_gemm_kernel<float>, smem);
        if (e_ != FERRIS_OK) return e_;
        ferris_launch(head_gemm_kernel<float>, grid, block, smem, s, (const float*)x, ldx, hsx, (const float*)w, (float*)out, ldo, hso,
                      (const float*)gate, ldg, tokens, K, N);
    } else if (dtype == FERRIS_BF16) {
        int e_ = ferris_allow_dynamic_smem((const void*)head_gemm_kernel<bf16>, smem);
        if (e_ != FERRIS_OK) return e_;
        ferris_launch(head_gemm_kernel<bf16>, grid, block, smem, s, (const bf16*)x, ldx, hsx, (const bf16*)w, (bf16*)out, ldo, hso,
                      (const bf16*)gate, ldg, tokens, K, N);
    } else
        FERRIS_REFUSE("head gemm: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}
