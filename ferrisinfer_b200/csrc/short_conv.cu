// A short causal convolution over time on each channel:
//   u_t[c] = a(r * y_t[c] + b[c] + sum_{j < taps} w[c, j] * y_(t - taps + 1 + j)[c]),   y before the sequence's start = 0,
// with r = 1 (the convolution is added to its own input) or 0, an optional bias b and a = nothing or SiLU.
// The taps - 1 inputs before a step's first token are the request's state ([slots, taps - 1, channels], fp32,
// oldest first; zero when the request is admitted), so a sequence may be cut into steps anywhere.
//
// Two launches.  `apply` is parallel over (token, channel) and only READS the state: a token whose tap reaches
// back before the step takes it from the state, otherwise from the step's own rows.  `advance` then moves the
// state on, one thread per (request, channel) walking the taps - 1 places in ascending order (with fewer new
// tokens than places, a place takes the value of a later place, which that thread has not overwritten yet).
// In one launch, a block that advanced the state could overtake a block that still reads it.  A step in which every
// request brings ONE token needs neither: one thread per (request, channel) reads the state, forms the output and
// shifts the state by one place, in one launch.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) short_conv_apply_kernel(
    const T* y, int ldy, T* __restrict__ out, int ldo, const float* __restrict__ w, const float* state,
    const int* __restrict__ token_seq, const int* __restrict__ positions, const int* __restrict__ seq_start_pos,
    const int* __restrict__ seq_state_slot, int channels, int taps, const float* __restrict__ bias, int residual, int act) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int seq = token_seq[t];
    const int pos = positions[t], start = seq_start_pos[seq];
    const int n = taps - 1;
    const float* st = state + (size_t)seq_state_slot[seq] * n * channels;
    const float own = to_float(y[(size_t)t * ldy + c]);
    float acc = (residual ? own : 0.0f) + (bias ? bias[c] : 0.0f);
    const float* wc = w + (size_t)c * taps;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        const int p = pos - back;
        float v;
        if (back == 0)
            v = own;
        else if (p < 0)
            v = 0.0f;
        else if (p >= start)
            v = to_float(y[(size_t)(t - back) * ldy + c]);
        else
            v = st[(size_t)(p - start + n) * channels + c];
        acc = fmaf(wc[j], v, acc);
    }
    if (act) acc = acc / (1.0f + expf(-acc));
    out[(size_t)t * ldo + c] = from_float<T>(acc);
}

template <typename T>
__global__ void __launch_bounds__(256) short_conv_advance_kernel(const T* y, int ldy, float* state,
                                                                 const int* __restrict__ seq_q_start,
                                                                 const int* __restrict__ seq_state_slot, int channels,
                                                                 int taps) {
    pdl_wait();
    pdl_launch_dependents();
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int n = taps - 1;
    const int row0 = seq_q_start[seq], len = seq_q_start[seq + 1] - row0;
    if (len <= 0) return;
    float* st = state + (size_t)seq_state_slot[seq] * n * channels;
    for (int k = 0; k < n; ++k) {
        const int idx = k + len;  // place in [the old state | the step's rows], of which the last n are kept
        st[(size_t)k * channels + c] = idx < n ? st[(size_t)idx * channels + c] : to_float(y[(size_t)(row0 + idx - n) * ldy + c]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) short_conv_single_kernel(const T* y, int ldy, T* __restrict__ out, int ldo,
                                                                const float* __restrict__ w, float* state,
                                                                const int* __restrict__ positions,
                                                                const int* __restrict__ seq_state_slot, int channels,
                                                                int taps, const float* __restrict__ bias, int residual,
                                                                int act) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;  // the request's only row of the step
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int n = taps - 1;
    const int pos = positions[t];
    float* st = state + (size_t)seq_state_slot[t] * n * channels + c;
    const float* wc = w + (size_t)c * taps;
    const float own = to_float(y[(size_t)t * ldy + c]);
    float acc = (residual ? own : 0.0f) + (bias ? bias[c] : 0.0f);
    for (int j = 0; j < n; ++j) {  // place j of the state is the input n - j positions back
        const float v = st[(size_t)j * channels];
        if (j > 0) st[(size_t)(j - 1) * channels] = v;
        acc = fmaf(wc[j], pos - (n - j) >= 0 ? v : 0.0f, acc);
    }
    acc = fmaf(wc[n], own, acc);
    if (n > 0) st[(size_t)(n - 1) * channels] = own;
    if (act) acc = acc / (1.0f + expf(-acc));
    out[(size_t)t * ldo + c] = from_float<T>(acc);
}

}  // namespace

// y, out: [tokens, channels] rows ldy / ldo apart (out must not be y); w: fp32 [channels, taps];
// state: fp32 [slots, taps - 1, channels] (may be null when taps == 1); bias: fp32 [channels] or null; residual: the
// input is added to the convolution; act: 0 nothing, 1 SiLU of the sum.
FERRIS_API int ferris_short_conv(const void* y, int ldy, void* out, int ldo, int dtype, const float* w, float* state,
                                 const int* token_seq, const int* positions, const int* seq_q_start,
                                 const int* seq_start_pos, const int* seq_state_slot, int tokens, int seqs, int channels,
                                 int taps, int advance, int single_tokens, const float* bias, int residual, int act,
                                 void* stream) {
    if (tokens <= 0 || seqs <= 0) return FERRIS_OK;
    if (channels <= 0 || taps <= 0) FERRIS_REFUSE("short conv: channels=%d taps=%d", channels, taps);
    if (taps > 1 && !state) FERRIS_REFUSE("short conv: %d taps need a state", taps);
    if (y == out) FERRIS_REFUSE("short conv: input and output must differ");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = channels >= 256 ? 256 : ((channels + 31) / 32) * 32;
    const int tiles = (channels + threads - 1) / threads;
    if (tiles > 65535) FERRIS_REFUSE("short conv: %d channels are more than one launch takes", channels);
    const dim3 block(threads), grid_a(tokens, tiles), grid_b(seqs, tiles);
    if (single_tokens && advance && tokens == seqs && dtype == FERRIS_F32) {
        ferris_launch(short_conv_single_kernel<float>, grid_a, block, 0, s, (const float*)y, ldy, (float*)out, ldo, w, state,
                      positions, seq_state_slot, channels, taps, bias, residual, act);
        FERRIS_LAUNCH_CHECK();
    }
    if (single_tokens && advance && tokens == seqs && dtype == FERRIS_BF16) {
        ferris_launch(short_conv_single_kernel<bf16>, grid_a, block, 0, s, (const bf16*)y, ldy, (bf16*)out, ldo, w, state,
                      positions, seq_state_slot, channels, taps, bias, residual, act);
        FERRIS_LAUNCH_CHECK();
    }
    if (dtype == FERRIS_F32) {
        ferris_launch(short_conv_apply_kernel<float>, grid_a, block, 0, s, (const float*)y, ldy, (float*)out, ldo, w,
                      (const float*)state, token_seq, positions, seq_start_pos, seq_state_slot, channels, taps, bias, residual, act);
        if (advance && taps > 1)
            ferris_launch(short_conv_advance_kernel<float>, grid_b, block, 0, s, (const float*)y, ldy, state, seq_q_start,
                          seq_state_slot, channels, taps);
    } else if (dtype == FERRIS_BF16) {
        ferris_launch(short_conv_apply_kernel<bf16>, grid_a, block, 0, s, (const bf16*)y, ldy, (bf16*)out, ldo, w,
                      (const float*)state, token_seq, positions, seq_start_pos, seq_state_slot, channels, taps, bias, residual, act);
        if (advance && taps > 1)
            ferris_launch(short_conv_advance_kernel<bf16>, grid_b, block, 0, s, (const bf16*)y, ldy, state, seq_q_start,
                          seq_state_slot, channels, taps);
    } else
        FERRIS_REFUSE("short conv: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}
