// Attention through a latent: what a token keeps is ONE row [c | r] for all heads, c a normed vector of `R`
// numbers from which every head's keys and values are linear maps (k_h = Uk_h c, v_h = Uv_h c), r a rotated key
// part of `dr` numbers that all heads share.  With a head's query split as [qn | qr], its score against token j is
//
//     s = (qn . Uk_h c_j + qr . r_j) * scale = ((Uk_h^T qn) . c_j + qr . r_j) * scale
//
// so a step's queries are first carried into the latent's space (`headwise_kernel`: qa = [Uk_h^T qn | turn(qr)]),
// every head then reads the same cached rows (`latent_attention_kernel`: scores against [c | r], the context
// as a weighted sum of c), and the head's value map is applied once to the context (`headwise_kernel`).  The
// cache is read once per token and step whatever the number of heads.  All arithmetic here is 32-bit; the cache
// rows and the value maps' outputs are in the storage type.
//
// Rotation: neighbours (2i, 2i+1) of the rotated part are turned by the token's angle i, (u, v) ->
// (u cos - v sin, v cos + u sin), cos and sin from the step's table times a constant magnitude.
#include "common.cuh"

// ------------------------------------------------------------------ the row a token keeps
// proj [N, ld] 32-bit, columns col0 .. col0 + R: the latent before its norm; the next dr: the shared key part.
// One block per token: c = x / sqrt(mean(x^2) + eps) * w, r turned; [c | r] to the token's place in the paged
// pool [pages, PAGE, R + dr] and, if asked for, to packed rows row_out [N, R + dr] (the step's own keys).
__global__ void __launch_bounds__(128) latent_kv_finish_kernel(const float* __restrict__ proj, int ld, int col0, int R, int dr,
                                                               int rot_dims, const float* __restrict__ w, float eps,
                                                               const float2* __restrict__ cs, int half, float mag,
                                                               T* __restrict__ pool, const int* __restrict__ table,
                                                               int table_stride, const int* __restrict__ token_seq,
                                                               const int* __restrict__ positions, const int* __restrict__ slots,
                                                               T* __restrict__ row_out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* x = proj + (size_t)t * ld + col0;
    float ss = 0.f;
    for (int d = threadIdx.x; d < R; d += blockDim.x) ss = fmaf(x[d], x[d], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)R + eps);
    const int pos = positions[t], slot = slots[token_seq[t]];
    const int page = table[(size_t)slot * table_stride + pos / IDM_PAGE];
    T* row = pool + ((size_t)page * IDM_PAGE + pos % IDM_PAGE) * (size_t)(R + dr);
    T* row2 = row_out ? row_out + (size_t)t * (R + dr) : nullptr;
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
        const float c = x[d] * inv * w[d];
        from_f32(row[d], c);
        if (row2) from_f32(row2[d], c);
    }
    const float* xr = x + R;
    for (int i = threadIdx.x; 2 * i < dr; i += blockDim.x) {
        float u = xr[2 * i], v = (2 * i + 1 < dr) ? xr[2 * i + 1] : 0.f;
        if (2 * i + 1 < rot_dims) {
            const float2 a = cs[(size_t)t * half + i];
            const float co = a.x * mag, si = a.y * mag;
            const float u2 = u * co - v * si, v2 = v * co + u * si;
            u = u2; v = v2;
        }
        from_f32(row[R + 2 * i], u);
        if (row2) from_f32(row2[R + 2 * i], u);
        if (2 * i + 1 < dr) {
            from_f32(row[R + 2 * i + 1], v);
            if (row2) from_f32(row2[R + 2 * i + 1], v);
        }
    }
}

extern "C" int idm_latent_kv_finish(const float* proj, int ld, int col0, int R, int dr, int rot_dims, const float* w,
                                    float eps, const float* cs, int half, float mag, void* pool, const int* table,
                                    int table_stride, const int* token_seq, const int* positions, const int* slots,
                                    void* row_out, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(R > 0 && dr >= 0 && col0 >= 0 && col0 + R + dr <= ld, "latent_kv_finish: columns %d + %d + %d of %d", col0, R, dr, ld);
    IDM_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 && (rot_dims == 0 || (cs != nullptr && half >= rot_dims / 2)),
                "latent_kv_finish: %d turned dims of %d with a table of %d angles", rot_dims, dr, half);
    idm_launch(latent_kv_finish_kernel, dim3(n_tokens), dim3(128), 0, stream, proj, ld, col0, R, dr, rot_dims, w, eps,
               (const float2*)cs, half, mag, (T*)pool, table, table_stride, token_seq, positions, slots, (T*)row_out);
    IDM_LAUNCH_CHECK("latent_kv_finish");
    return 0;
}

// ------------------------------------------------------------------ a matrix per head
// out[t, h, o] = sum_i x[t, h, i] * W[h, i, o] for every head h on its own: x 32-bit with strides of its own, W
// [H, I, O] in the storage type (o contiguous: a thread owns an output and reads W side by side with its
// neighbours), sums in 32-bit in ascending i.  `tail` more columns of x behind the I are copied behind the O
// outputs, the first `rot_dims` of them turned by the token's angles (a query's rotated part).  A block has one
// head and up to HW_TOKENS tokens, so a head's matrix is read once per that many tokens.
#define HW_TOKENS 8

template <typename OutT>
__global__ void __launch_bounds__(128) headwise_kernel(const float* __restrict__ x, long long x_tok, int x_head, int I,
                                                       const T* __restrict__ W, int O, OutT* __restrict__ out,
                                                       long long o_tok, int o_head, int tail, int rot_dims,
                                                       const float2* __restrict__ cs, int half, float mag, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];                       // [HW_TOKENS][I]
    const int h = blockIdx.y, t0 = blockIdx.x * HW_TOKENS;
    const int nt = min(HW_TOKENS, n_tokens - t0);
    for (int e = threadIdx.x; e < nt * I; e += blockDim.x) {
        const int tt = e / I, i = e % I;
        xs[tt * I + i] = x[(size_t)(t0 + tt) * x_tok + (size_t)h * x_head + i];
    }
    __syncthreads();
    const T* Wh = W + (size_t)h * I * O;
    for (int o = threadIdx.x; o < O; o += blockDim.x) {
        float acc[HW_TOKENS];
#pragma unroll
        for (int tt = 0; tt < HW_TOKENS; ++tt) acc[tt] = 0.f;
        for (int i = 0; i < I; ++i) {
            const float wv = to_f32(Wh[(size_t)i * O + o]);
#pragma unroll
            for (int tt = 0; tt < HW_TOKENS; ++tt) acc[tt] = fmaf(xs[tt * I + i], wv, acc[tt]);   // (rows past nt: unused)
        }
#pragma unroll
        for (int tt = 0; tt < HW_TOKENS; ++tt)
            if (tt < nt) from_f32(out[(size_t)(t0 + tt) * o_tok + (size_t)h * o_head + o], acc[tt]);
    }
    for (int e = threadIdx.x; e < nt * ((tail + 1) / 2); e += blockDim.x) {
        const int tt = e / ((tail + 1) / 2), i = e % ((tail + 1) / 2), t = t0 + tt;
        const float* xr = x + (size_t)t * x_tok + (size_t)h * x_head + I;
        OutT* orow = out + (size_t)t * o_tok + (size_t)h * o_head + O;
        float u = xr[2 * i], v = (2 * i + 1 < tail) ? xr[2 * i + 1] : 0.f;
        if (2 * i + 1 < rot_dims) {
            const float2 a = cs[(size_t)t * half + i];
            const float co = a.x * mag, si = a.y * mag;
            const float u2 = u * co - v * si, v2 = v * co + u * si;
            u = u2; v = v2;
        }
        from_f32(orow[2 * i], u);
        if (2 * i + 1 < tail) from_f32(orow[2 * i + 1], v);
    }
}

// out_is_f32: the outputs are 32-bit (queries in the latent's space); else the storage type (a product's input)
extern "C" int idm_headwise(const float* x, long long x_tok, int x_head, int I, const void* W, int O, void* out,
                            int out_is_f32, long long o_tok, int o_head, int tail, int rot_dims, const float* cs, int half,
                            float mag, int n_tokens, int n_heads, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(I > 0 && O >= 0 && n_heads > 0 && tail >= 0, "headwise: sizes I=%d O=%d heads=%d tail=%d", I, O, n_heads, tail);
    IDM_REQUIRE(rot_dims >= 0 && rot_dims <= tail && rot_dims % 2 == 0 && (rot_dims == 0 || (cs != nullptr && half >= rot_dims / 2)),
                "headwise: %d turned dims of %d with a table of %d angles", rot_dims, tail, half);
    const size_t smem = (size_t)HW_TOKENS * I * sizeof(float);
    IDM_REQUIRE(smem <= 200 * 1024, "headwise: I=%d does not fit shared memory", I);
    const dim3 grid((n_tokens + HW_TOKENS - 1) / HW_TOKENS, n_heads);
    if (out_is_f32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(headwise_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        idm_launch(headwise_kernel<float>, grid, dim3(128), smem, stream, x, x_tok, x_head, I, (const T*)W, O, (float*)out,
                   o_tok, o_head, tail, rot_dims, (const float2*)cs, half, mag, n_tokens);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(headwise_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        idm_launch(headwise_kernel<T>, grid, dim3(128), smem, stream, x, x_tok, x_head, I, (const T*)W, O, (T*)out,
                   o_tok, o_head, tail, rot_dims, (const float2*)cs, half, mag, n_tokens);
    }
    IDM_LAUNCH_CHECK("headwise");
    return 0;
}

// ------------------------------------------------------------------ attention over the latent rows
// A block has one query token, up to LA_WARPS heads (a warp each) and one run of keys: positions
// [run * run_keys, (run + 1) * run_keys) up to the query's own.  Keys are walked in blocks of 32 at absolute
// positions, staged in shared memory once for all the block's heads; lane i scores key j0 + i against the head's
// query (kept in shared memory, 32-bit), the running (max, sum, context) is rescaled block by block, and the
// context is a weighted sum of the rows' first R numbers, a lane owning pairs of neighbours.  With one run the
// block finishes the row (the sink, a score with no key and no value, joins the sum once) and writes the context
// [N, H, R] in 32-bit; with several, every run leaves (max, sum, context) in scratch and latent_fold_kernel adds
// the runs in ascending order.
#define LA_WARPS 8

struct LatentArgs {
    const float* qa;          // [N, H, D]
    const T* pool;            // [pages, PAGE, D]
    const int* table; int table_stride;
    const int* token_seq; const int* positions; const int* slots;
    const float* sink;        // [H] or null
    float* ctx;               // [N, H, R]
    float* part;              // [N, H, n_runs, R + 2]: (max, sum, context) of each run
    int n_tokens, H, R, D;
    float scale;
    int run_keys, n_runs, stride_words;
};

template <int NACC>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(LatentArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* qs = reinterpret_cast<float*>(smem_raw);                          // [LA_WARPS][D] (rows padded to 4 floats)
    const int Dq = (a.D + 3) & ~3;
    uint32_t* tile = reinterpret_cast<uint32_t*>(qs + LA_WARPS * Dq);        // [32][stride_words]
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, head = blockIdx.y * LA_WARPS + wib, run = blockIdx.z;
    const bool live_head = head < a.H;
    const int pos = a.positions[t], slot = a.slots[a.token_seq[t]];
    const int lo = run * a.run_keys, hi = min(pos, lo + a.run_keys - 1);      // keys lo .. hi
    float m = -INFINITY, l = 0.f;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    if (lo <= pos) {
        if (live_head) {
            const float* q = a.qa + ((size_t)t * a.H + head) * a.D;
            for (int d = lane; d < Dq; d += 32) qs[wib * Dq + d] = d < a.D ? q[d] : 0.f;
        }
        const int row_bytes = a.D * (int)sizeof(T);
        const bool vec = (row_bytes % 16) == 0;
        const int* pages = a.table + (size_t)slot * a.table_stride;
        for (int j0 = lo; j0 <= hi; j0 += 32) {
            __syncthreads();                                                  // the last block's readers are done (and qs is written)
            const int nk = min(32, hi - j0 + 1);
            if (vec) {
                const int cpr = row_bytes / 16;
                for (int c = threadIdx.x; c < nk * cpr; c += LA_WARPS * 32) {
                    const int r = c / cpr, cc = c % cpr, j = j0 + r;
                    const T* src = a.pool + ((size_t)pages[j / IDM_PAGE] * IDM_PAGE + j % IDM_PAGE) * (size_t)a.D;
                    *reinterpret_cast<uint4*>(tile + (size_t)r * a.stride_words + cc * 4) = *(reinterpret_cast<const uint4*>(src) + cc);
                }
            } else {
                T* tl = reinterpret_cast<T*>(tile);
                const int stride_e = a.stride_words * 4 / (int)sizeof(T);
                for (int c = threadIdx.x; c < nk * a.D; c += LA_WARPS * 32) {
                    const int r = c / a.D, d = c % a.D, j = j0 + r;
                    tl[(size_t)r * stride_e + d] = a.pool[((size_t)pages[j / IDM_PAGE] * IDM_PAGE + j % IDM_PAGE) * (size_t)a.D + d];
                }
            }
            __syncthreads();
            if (!live_head) continue;
            const bool valid = lane < nk;
            float sc = -INFINITY;
            if (valid) {
                const T* krow = reinterpret_cast<const T*>(tile + (size_t)lane * a.stride_words);
                const float* q = qs + wib * Dq;
                float d0 = 0.f, d1 = 0.f;
                constexpr int VN = Vec16<T>::N;
                int d = 0;
                for (; d + VN <= a.D; d += VN) {
                    Vec16<T> kv; kv.load(krow + d);
#pragma unroll
                    for (int e = 0; e < VN; e += 2) {
                        d0 = fmaf(q[d + e], kv.get(e), d0);
                        d1 = fmaf(q[d + e + 1], kv.get(e + 1), d1);
                    }
                }
                for (; d < a.D; ++d) d0 = fmaf(q[d], to_f32(krow[d]), d0);
                sc = (d0 + d1) * a.scale;
            }
            const float m_new = fmaxf(m, warp_max(sc));
            const float alpha = expf(m - m_new);                              // (m = -inf at first: 0)
            const float p = valid ? expf(sc - m_new) : 0.f;
            l = l * alpha + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
            for (int jj = 0; jj < nk; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const T* crow = reinterpret_cast<const T*>(tile + (size_t)jj * a.stride_words);
#pragma unroll
                for (int i = 0; i < NACC / 2; ++i) {
                    const int d = 2 * lane + 64 * i;
                    if (d < a.R) {                                            // (d + 1 may be R: inside the row, never stored)
                        float c0, c1;
                        if (sizeof(T) == 2) {
                            const uint32_t wv = *reinterpret_cast<const uint32_t*>(crow + d);
                            c0 = __uint_as_float(wv << 16); c1 = __uint_as_float(wv & 0xffff0000u);
                        } else {
                            const float2 cv = *reinterpret_cast<const float2*>(crow + d);
                            c0 = cv.x; c1 = cv.y;
                        }
                        acc[2 * i] = fmaf(pj, c0, acc[2 * i]);
                        acc[2 * i + 1] = fmaf(pj, c1, acc[2 * i + 1]);
                    }
                }
            }
        }
    }
    if (!live_head) return;
    if (a.n_runs == 1) {
        const float sk = a.sink ? a.sink[head] : -INFINITY;
        const float mf = fmaxf(m, sk);
        const float w = expf(m - mf);
        const float inv = 1.0f / (l * w + (a.sink ? expf(sk - mf) : 0.f));
        float* o = a.ctx + ((size_t)t * a.H + head) * a.R;
#pragma unroll
        for (int i = 0; i < NACC / 2; ++i) {
            const int d = 2 * lane + 64 * i;
            if (d < a.R) o[d] = acc[2 * i] * w * inv;
            if (d + 1 < a.R) o[d + 1] = acc[2 * i + 1] * w * inv;
        }
    } else {
        float* o = a.part + (((size_t)t * a.H + head) * a.n_runs + run) * (size_t)(a.R + 2);
        if (lane == 0) { o[0] = m; o[1] = l; }
        if (lo <= pos) {
#pragma unroll
            for (int i = 0; i < NACC / 2; ++i) {
                const int d = 2 * lane + 64 * i;
                if (d < a.R) o[2 + d] = acc[2 * i];
                if (d + 1 < a.R) o[2 + d + 1] = acc[2 * i + 1];
            }
        }
    }
}

// one warp per (token, head): the runs' results in ascending order, then the sink
__global__ void __launch_bounds__(128) latent_fold_kernel(const float* __restrict__ part, const float* __restrict__ sink,
                                                          float* __restrict__ ctx, const int* __restrict__ positions,
                                                          int n_tokens, int H, int R, int run_keys, int n_runs) {
    pdl_launch_dependents();
    pdl_wait();
    const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (long long)n_tokens * H) return;
    const int t = (int)(w / H), head = (int)(w % H);
    const int used = min(n_runs, positions[t] / run_keys + 1);               // runs that hold keys of this query
    const float* p = part + (size_t)w * n_runs * (R + 2);
    const float sk = sink ? sink[head] : -INFINITY;
    float mf = sk;
    for (int r = 0; r < used; ++r) mf = fmaxf(mf, p[(size_t)r * (R + 2)]);
    float l = 0.f;
    for (int r = 0; r < used; ++r) l += p[(size_t)r * (R + 2) + 1] * expf(p[(size_t)r * (R + 2)] - mf);
    if (sink) l += expf(sk - mf);
    const float inv = 1.0f / l;
    float* o = ctx + (size_t)w * R;
    for (int d = lane; d < R; d += 32) {
        float s = 0.f;
        for (int r = 0; r < used; ++r) s = fmaf(p[(size_t)r * (R + 2) + 2 + d], expf(p[(size_t)r * (R + 2)] - mf), s);
        o[d] = s * inv;
    }
}

extern "C" int idm_latent_attention_max_rank() { return 1024; }

// run_keys: a multiple of 32; n_runs * run_keys covers every position of the step (n_runs == 1: no scratch)
extern "C" int idm_latent_attention(const float* qa, const void* pool, const int* table, int table_stride,
                                    const int* token_seq, const int* positions, const int* slots, const float* sink,
                                    float* ctx, float* part, int n_tokens, int H, int R, int D, float scale,
                                    int run_keys, int n_runs, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(H > 0 && R > 0 && D >= R && R <= 1024, "latent_attention: heads=%d rank=%d row=%d (rank at most 1024)", H, R, D);
    IDM_REQUIRE(n_runs >= 1 && run_keys > 0 && run_keys % 32 == 0 && (n_runs == 1 || part != nullptr),
                "latent_attention: %d runs of %d keys", n_runs, run_keys);
    LatentArgs a;
    a.qa = qa; a.pool = (const T*)pool; a.table = table; a.table_stride = table_stride;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots; a.sink = sink; a.ctx = ctx; a.part = part;
    a.n_tokens = n_tokens; a.H = H; a.R = R; a.D = D; a.scale = scale; a.run_keys = run_keys; a.n_runs = n_runs;
    // a row of the staged block: whole 16-byte pieces, and a stride of 4 (mod 8) words, so that eight lanes that
    // read 16 bytes each at the same column of eight rows touch every bank once
    int words = (D * (int)sizeof(T) + 15) / 16 * 4;
    while (words % 8 != 4) words += 4;
    a.stride_words = words;
    const size_t smem = (size_t)LA_WARPS * ((D + 3) & ~3) * sizeof(float) + (size_t)32 * words * 4;
    IDM_REQUIRE(smem <= 220 * 1024, "latent_attention: rows of %d do not fit shared memory", D);
    const dim3 grid(n_tokens, (H + LA_WARPS - 1) / LA_WARPS, n_runs);
    IDM_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "latent_attention: grid %d x %d", grid.y, grid.z);
#define LA_LAUNCH(NACC)                                                                                              \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(latent_attention_kernel<NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        idm_launch(latent_attention_kernel<NACC>, grid, dim3(LA_WARPS * 32), smem, stream, a);                       \
    } while (0)
    if (R <= 64) LA_LAUNCH(2);
    else if (R <= 128) LA_LAUNCH(4);
    else if (R <= 256) LA_LAUNCH(8);
    else if (R <= 512) LA_LAUNCH(16);
    else LA_LAUNCH(32);
#undef LA_LAUNCH
    IDM_LAUNCH_CHECK("latent_attention");
    if (n_runs > 1) {
        const long long warps = (long long)n_tokens * H;
        idm_launch(latent_fold_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, (const float*)part, sink, ctx,
                   positions, n_tokens, H, R, run_keys, n_runs);
        IDM_LAUNCH_CHECK("latent_fold");
    }
    return 0;
}

// ------------------------------------------------------------------ whole prompts: keys and values per head
// A step that brings whole prompts (every sequence from its first token) has more queries than heads' worth of
// latent space pays for: there the keys and values are made per head from the step's rows once, k_h = [Uk_h c | r]
// and v_h = Uv_h c, and the step runs the attention kernel for heads with keys and values of their own.  This
// kernel lays its operands out: q [N, H, hd] = [qn | turn(qr) | 0], and pages of their own [pages, H, PAGE, hd]
// for k and v (0 behind a head's own dims), addressed through a block table of the step's own.
// proj: the joint projection (a head's query at column h * (dn + dr)); up: [N, H * dn + H * dv] = the rows' c times
// [Uk ; Uv]; rows: the step's packed [c | r] rows in the storage type.  One block per token.
__global__ void __launch_bounds__(256) latent_expand_pack_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ up,
                                                                 const T* __restrict__ rows, int H, int dn, int dr, int dv, int R,
                                                                 int rot_dims, const float2* __restrict__ cs, int half, float mag,
                                                                 int hd, T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                                                 const int* __restrict__ table, int table_stride,
                                                                 const int* __restrict__ token_seq, const int* __restrict__ positions,
                                                                 const int* __restrict__ slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t], slot = slots[token_seq[t]];
    const int page = table[(size_t)slot * table_stride + pos / IDM_PAGE];
    const float* pq = proj + (size_t)t * ld;
    const float* pu = up + (size_t)t * (size_t)(H * dn + H * dv);
    const T* r = rows + (size_t)t * (R + dr) + R;
    for (int e = threadIdx.x; e < H * hd; e += blockDim.x) {
        const int h = e / hd, d = e % hd;
        float qv = 0.f;
        T kk, vv;
        from_f32(kk, 0.f); from_f32(vv, 0.f);
        if (d < dn) {
            qv = pq[h * (dn + dr) + d];
            from_f32(kk, pu[h * dn + d]);
        } else if (d < dn + dr) {
            const int j = d - dn;
            const float* qr = pq + h * (dn + dr) + dn;
            qv = qr[j];
            if ((j | 1) < rot_dims) {                       // the pair (j & ~1, j | 1) is turned
                const float2 a = cs[(size_t)t * half + (j >> 1)];
                const float co = a.x * mag, si = a.y * mag;
                qv = (j & 1) ? qr[j] * co + qr[j - 1] * si : qr[j] * co - qr[j + 1] * si;
            }
            kk = r[j];
        }
        if (d < dv) from_f32(vv, pu[H * dn + h * dv + d]);
        from_f32(q[((size_t)t * H + h) * hd + d], qv);
        const size_t at = (((size_t)page * H + h) * IDM_PAGE + pos % IDM_PAGE) * hd + d;
        k[at] = kk;
        v[at] = vv;
    }
}

extern "C" int idm_latent_expand_pack(const float* proj, int ld, const float* up, const void* rows, int H, int dn, int dr,
                                      int dv, int R, int rot_dims, const float* cs, int half, float mag, int hd, void* q,
                                      void* k, void* v, const int* table, int table_stride, const int* token_seq,
                                      const int* positions, const int* slots, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(H > 0 && dn >= 0 && dr >= 0 && dv > 0 && dn + dr <= hd && dv <= hd, "latent_expand_pack: heads of %d + %d and %d in %d",
                dn, dr, dv, hd);
    IDM_REQUIRE(rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 && (rot_dims == 0 || (cs != nullptr && half >= rot_dims / 2)),
                "latent_expand_pack: %d turned dims of %d with a table of %d angles", rot_dims, dr, half);
    idm_launch(latent_expand_pack_kernel, dim3(n_tokens), dim3(256), 0, stream, proj, ld, up, (const T*)rows, H, dn, dr, dv, R, rot_dims,
               (const float2*)cs, half, mag, hd, (T*)q, (T*)k, (T*)v, table, table_stride, token_seq, positions, slots);
    IDM_LAUNCH_CHECK("latent_expand_pack");
    return 0;
}
