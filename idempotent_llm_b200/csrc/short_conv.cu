// Short causal convolutions over time with per-sequence state, for mixers that filter their
// projections channel by channel:
//
//   y[t, c] = sum_j w[c, j] * u[t - taps + 1 + j, c]      (j = 0 .. taps - 1; zeros before the sequence's start)
//
// u are columns [col0, col0 + channels) of a 32-bit projection [N, in_stride] of the step's packed tokens.
// Inputs before the step's first token come from the sequence's state: `taps - 1` rows of `channels`
// floats per slot, holding the inputs at positions q_start - taps + 1 .. q_start - 1.  The sum runs in
// ascending j in 32-bit whatever the step looks like, so a token's result does not depend on how its
// sequence was cut into steps.
//
// State is moved on behind the reads: a sequence that brings one token has its rows shifted by the thread
// that owns the channel (it has read all of them); sequences that bring more are moved on by
// conv_state_update_kernel, launched after every reader of the old state.
#include "common.cuh"

#define CONV_MAX_TAPS 8

struct ConvSeg {
    const float* in; int in_stride; int col0;       // projection of the step [N, in_stride], first column
    int channels, taps;
    const float* w;                                 // [channels, taps]
    const float* bias;                              // [channels] or null
    float* state; long long state_stride;           // state + slot * state_stride : [taps - 1, channels]
};

struct ConvStep {
    const int* token_seq; const int* positions; const int* slots; const int* q_start; const int* cu_q;
};

// what a token's filters need to know of its sequence: looked up once per thread (or block)
struct ConvToken {
    int pos;        // the token's position
    int avail;      // tokens of this step before it in its sequence: inputs further back come from the state
    int slot;
    int single;     // its sequence brings this token only: the filter moves the state on itself
};
__device__ __forceinline__ ConvToken conv_token(const ConvStep& st, int t) {
    const int s = st.token_seq[t];
    ConvToken m;
    m.pos = st.positions[t];
    m.avail = m.pos - st.q_start[s];
    m.slot = st.slots[s];
    m.single = st.cu_q[s + 1] - st.cu_q[s] == 1;
    return m;
}

// the convolution of token t, channel c (the number of taps known at compile time: the loops unroll to straight
// code); moves the state on if t is its sequence's only token
template <int TAPS>
__device__ __forceinline__ float conv_at(const ConvSeg& g, const ConvToken& m, int t, int c) {
    constexpr int H = TAPS - 1;
    const float* base = g.in + (size_t)t * g.in_stride + g.col0 + c;
    float* srow = g.state + (size_t)m.slot * g.state_stride + c;
    float u[TAPS];
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
        const int back = H - j;                                    // the input `back` positions before the token
        float v = 0.f;
        if (back <= m.avail) v = base[-(ptrdiff_t)back * g.in_stride];
        else if (back <= m.pos) v = srow[(size_t)(H - (back - m.avail)) * g.channels];
        u[j] = v;
    }
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) acc = fmaf(g.w[(size_t)c * TAPS + j], u[j], acc);
    if (g.bias) acc += g.bias[c];
    if (m.single) {
#pragma unroll
        for (int j = 1; j < TAPS; ++j) srow[(size_t)(j - 1) * g.channels] = u[j];
    }
    return acc;
}

// silu of a filter's output: exact in the 32-bit library; with the hardware exponential and division where the
// result is rounded to bfloat16 operands anyway (relative error ~1e-6)
__device__ __forceinline__ float silu_exact(float v) {
#if defined(IDM_F32)
    return v / (1.0f + expf(-v));
#else
    return __fdividef(v, 1.0f + __expf(-v));
#endif
}

// out [N, channels] 32-bit; act: 0 none, 1 silu
template <int TAPS>
__global__ void __launch_bounds__(256) short_conv_kernel(ConvSeg g, ConvStep st, float* __restrict__ out, int act) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ ConvToken token;                     // (one token per block: looked up by one thread)
    const int c = blockIdx.y * blockDim.x + threadIdx.x, t = blockIdx.x;
    if (threadIdx.x == 0) token = conv_token(st, t);
    __syncthreads();
    if (c >= g.channels) return;
    const float v = conv_at<TAPS>(g, token, t, c);
    out[(size_t)t * g.channels + c] = act == 1 ? silu_exact(v) : v;
}

// The attention side: q, k and v channels [n_q * dk | n_kv * dk | n_kv * dv] are filtered, the first
// 2 * half dims of every q and k head turned by the token's position (dim i with dim i + half; (u, v) ->
// (u cos - v sin, v cos + u sin), table cs [N, half] of (cos, sin)), q stored [N, n_q, dk] and k, v written
// to the token's place in the cache (pools [pages, n_kv, PAGE, dk] and [pages, n_kv, PAGE, dv]).
struct ConvQkvArgs {
    ConvSeg seg; ConvStep st;
    int n_q, n_kv, dk, dv, half;
    const float2* cs;
    T* q_out; T* k_pool; T* v_pool;
    const int* table; int table_stride;
};

template <int TAPS>
__global__ void __launch_bounds__(256) conv_qkv_cache_kernel(ConvQkvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const ConvToken m = conv_token(a.st, t);                       // (one token per block: every thread the same)
    const size_t page = a.table[(size_t)m.slot * a.table_stride + m.pos / IDM_PAGE], prow = m.pos % IDM_PAGE;
    const int qk_heads = a.n_q + a.n_kv;
    const int rest = a.dk - a.half;                       // work items of a q or k head: pairs, then single dims
    const int qk_items = qk_heads * rest, v_items = a.n_kv * a.dv;
    // (steps of few tokens spread a token's items over several blocks: gridDim.y)
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < qk_items + v_items; i += gridDim.y * blockDim.x) {
        if (i < qk_items) {
            const int head = i / rest, r = i % rest;
            T* dst = head < a.n_q ? a.q_out + ((size_t)t * a.n_q + head) * a.dk
                                  : a.k_pool + ((page * a.n_kv + (head - a.n_q)) * IDM_PAGE + prow) * (size_t)a.dk;
            if (r < a.half) {
                const float u = conv_at<TAPS>(a.seg, m, t, head * a.dk + r);
                const float v = conv_at<TAPS>(a.seg, m, t, head * a.dk + r + a.half);
                const float2 cs = a.cs[(size_t)t * a.half + r];
                from_f32(dst[r], u * cs.x - v * cs.y);
                from_f32(dst[r + a.half], v * cs.x + u * cs.y);
            } else {
                const int d = r + a.half;
                from_f32(dst[d], conv_at<TAPS>(a.seg, m, t, head * a.dk + d));
            }
        } else {
            const int j = i - qk_items, g = j / a.dv, d = j % a.dv;
            T* dst = a.v_pool + ((page * a.n_kv + g) * IDM_PAGE + prow) * (size_t)a.dv;
            from_f32(dst[d], conv_at<TAPS>(a.seg, m, t, qk_heads * a.dk + j));
        }
    }
}

// After every reader: the state of sequences that brought more than one token becomes the inputs at their
// last taps - 1 positions.  One thread per (sequence, channel) reads its rows, then writes them.
__global__ void __launch_bounds__(256) conv_state_update_kernel(ConvSeg g, ConvStep st, const int* __restrict__ kv_len) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (c >= g.channels) return;
    const int n_new = st.cu_q[s + 1] - st.cu_q[s];
    if (n_new <= 1) return;                          // (one token: moved on by the convolution itself)
    const int start = st.q_start[s], end = kv_len[s], hist = g.taps - 1;
    float* srow = g.state + (size_t)st.slots[s] * g.state_stride + c;
    float u[CONV_MAX_TAPS];
#pragma unroll
    for (int r = 0; r < CONV_MAX_TAPS - 1; ++r) {
        if (r >= hist) break;
        const int p = end - hist + r;
        float v = 0.f;
        if (p >= start) v = g.in[(size_t)(st.cu_q[s] + p - start) * g.in_stride + g.col0 + c];
        else if (p >= 0) v = srow[(size_t)(p - (start - hist)) * g.channels];
        u[r] = v;
    }
#pragma unroll
    for (int r = 0; r < CONV_MAX_TAPS - 1; ++r) {
        if (r >= hist) break;
        srow[(size_t)r * g.channels] = u[r];
    }
}

static int conv_seg(ConvSeg& g, const char* what, const float* in, int in_stride, int col0, int channels, int taps,
                    const float* w, const float* bias, float* state, long long state_stride) {
    IDM_REQUIRE(channels > 0 && taps >= 1 && taps <= CONV_MAX_TAPS, "%s: %d channels, %d taps (at most %d)", what, channels,
                taps, CONV_MAX_TAPS);
    IDM_REQUIRE(col0 >= 0 && col0 + channels <= in_stride, "%s: columns %d..%d of rows of %d", what, col0, col0 + channels, in_stride);
    IDM_REQUIRE(taps == 1 || (state != nullptr && state_stride >= (long long)(taps - 1) * channels),
                "%s: the state of a slot must hold %d rows of %d floats", what, taps - 1, channels);
    g.in = in; g.in_stride = in_stride; g.col0 = col0; g.channels = channels; g.taps = taps; g.w = w; g.bias = bias;
    g.state = state; g.state_stride = state_stride;
    return 0;
}

extern "C" int idm_short_conv(const float* in, int in_stride, int col0, int channels, int taps, const float* w,
                              const float* bias, int act, float* state, long long state_stride, float* out,
                              const int* token_seq, const int* positions, const int* slots, const int* q_start,
                              const int* cu_q, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    ConvSeg g;
    if (conv_seg(g, "short_conv", in, in_stride, col0, channels, taps, w, bias, state, state_stride)) return 1;
    ConvStep st{token_seq, positions, slots, q_start, cu_q};
    const dim3 grid(n_tokens, (channels + 255) / 256);
#define CONV_GO(TAPS_) case TAPS_: idm_launch(short_conv_kernel<TAPS_>, grid, dim3(256), 0, stream, g, st, out, act); break;
    switch (taps) { CONV_GO(1) CONV_GO(2) CONV_GO(3) CONV_GO(4) CONV_GO(5) CONV_GO(6) CONV_GO(7) CONV_GO(8) }
#undef CONV_GO
    IDM_LAUNCH_CHECK("short_conv");
    return 0;
}

extern "C" int idm_conv_qkv_cache(const float* in, int in_stride, int col0, int taps, const float* w, float* state,
                                  long long state_stride, int n_q, int n_kv, int dk, int dv, int half, const float* cs,
                                  void* q_out, void* k_pool, void* v_pool, const int* table, int table_stride,
                                  const int* token_seq, const int* positions, const int* slots, const int* q_start,
                                  const int* cu_q, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    ConvQkvArgs a;
    const int channels = (n_q + n_kv) * dk + n_kv * dv;
    if (conv_seg(a.seg, "conv_qkv_cache", in, in_stride, col0, channels, taps, w, nullptr, state, state_stride)) return 1;
    IDM_REQUIRE(n_q > 0 && n_kv > 0 && dk > 0 && dv > 0 && half >= 0 && 2 * half <= dk,
                "conv_qkv_cache: heads %d/%d, sizes %d/%d, %d turning pairs", n_q, n_kv, dk, dv, half);
    IDM_REQUIRE(half == 0 || cs != nullptr, "conv_qkv_cache: a rotation needs its table");
    a.st = ConvStep{token_seq, positions, slots, q_start, cu_q};
    a.n_q = n_q; a.n_kv = n_kv; a.dk = dk; a.dv = dv; a.half = half; a.cs = (const float2*)cs;
    a.q_out = (T*)q_out; a.k_pool = (T*)k_pool; a.v_pool = (T*)v_pool; a.table = table; a.table_stride = table_stride;
    // a block per token; with few tokens, several blocks per token, so that two blocks' worth of work per SM is about
    const int items = (n_q + n_kv) * (dk - half) + n_kv * dv;
    int split = (296 + n_tokens - 1) / n_tokens;
    if (split > (items + 255) / 256) split = (items + 255) / 256;
    if (split < 1) split = 1;
    const dim3 grid(n_tokens, split);
#define CONV_GO(TAPS_) case TAPS_: idm_launch(conv_qkv_cache_kernel<TAPS_>, grid, dim3(256), 0, stream, a); break;
    switch (taps) { CONV_GO(1) CONV_GO(2) CONV_GO(3) CONV_GO(4) CONV_GO(5) CONV_GO(6) CONV_GO(7) CONV_GO(8) }
#undef CONV_GO
    IDM_LAUNCH_CHECK("conv_qkv_cache");
    return 0;
}

extern "C" int idm_conv_state_update(const float* in, int in_stride, int col0, int channels, int taps, float* state,
                                     long long state_stride, const int* slots, const int* q_start, const int* cu_q,
                                     const int* kv_len, int n_seqs, cudaStream_t stream) {
    if (n_seqs == 0 || taps <= 1) return 0;
    ConvSeg g;
    if (conv_seg(g, "conv_state_update", in, in_stride, col0, channels, taps, nullptr, nullptr, state, state_stride)) return 1;
    IDM_REQUIRE(n_seqs <= 65535, "conv_state_update: %d sequences in one launch", n_seqs);
    ConvStep st{nullptr, nullptr, slots, q_start, cu_q};
    idm_launch(conv_state_update_kernel, dim3((channels + 255) / 256, n_seqs), dim3(256), 0, stream, g, st, kv_len);
    IDM_LAUNCH_CHECK("conv_state_update");
    return 0;
}
