// The gated delta rule: a linear recurrence with one matrix of state per head, S [dk, dv] in float32, which a token
// first lets decay, then corrects along its key towards its value, then reads with its query:
//
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q        (g, beta: one number per head and token)
//
// Every column of S (one value dimension) goes through this on its own, so columns are spread over threads and a
// request's tokens are taken in order; nothing but q, k, g and beta is shared between columns.
//
// Kernels, in the order a step runs them:
//   gdr_prepare      per (token, head of q, k or v): add the projection's split-K shares, the short causal convolution
//                    over time with its SiLU (inputs before the portion's start come from the request's kept tail),
//                    q and k made unit vectors per head (q also times `q_scale`), beta = sigmoid,
//                    g = exp(-exp(A_log) * softplus(a + dt_bias)); all float32
//   gdr_conv_tail    per request: the last taps-1 convolution inputs of the step become the kept tail
//   gdr_recurrent    per (request, head, a few columns): the recurrence over the step's tokens, state in registers, 16
//                    (or 32) lanes a column.  Both products with the state are taken from the state before the
//                    token's update, a = S^T k and b = S^T q, so that they share one exchange between the lanes:
//                    u = beta (v - g a), o = g b + u (k . q), S <- g S + k u^T, which is the same arithmetic; and two
//                    tokens are taken at a time, the second one's products following from the first one's correction
//   gdr_out_norm     per (token, head): o / rms(o) * weight * silu(gate), rounded to the engine's dtype
//
// A request's slot of state is one float32 array: S as [heads][dv][dk] (a column's dk values side by side), then the
// tail as [taps-1][channels]
// (oldest first).  Projection rows are [q: G*dk | k: G*dk | v: H*dv | b: H | a: H | gate: H*dv]; head h of H reads
// q/k head h / (H / G).
#include "common.cuh"

__device__ __forceinline__ float gdr_slab_sum(const float* row, int c, int n_partials, long partial_stride) {
    float v = row[c];
    for (int p = 1; p < n_partials; ++p) v += row[(size_t)p * partial_stride + c];
    return v;
}
__device__ __forceinline__ float gdr_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float gdr_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <typename TW>
__global__ void __launch_bounds__(128)
gdr_prepare_kernel(const float* __restrict__ proj, long proj_stride, int n_partials, long partial_stride,
                   const TW* __restrict__ conv_w, int taps, const TW* __restrict__ a_log, const TW* __restrict__ dt_bias,
                   const float* __restrict__ state, long state_stride, long tail_off, const int* __restrict__ row_seq,
                   const int* __restrict__ seq_q_start, const int* __restrict__ seq_slot, float* __restrict__ qkv,
                   float* __restrict__ beta, float* __restrict__ decay, int G, int H, int dk, int dv, float q_scale,
                   float unit_eps) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    constexpr int PER = 8;                             // channels a thread takes: heads of up to 1024
    __shared__ float red[32];
    const int row = blockIdx.x, unit = blockIdx.y, tid = threadIdx.x;
    const int qk = G * dk, C = 2 * qk + H * dv;
    const bool is_v = unit >= 2 * G;
    const int width = is_v ? dv : dk;
    const int base = is_v ? 2 * qk + (unit - 2 * G) * dv : unit * dk;    // q heads, then k heads, then v heads
    const int seq = row_seq[row];
    const int i = row - seq_q_start[seq];              // place within the step's portion of this request
    const float* tail = state + (size_t)seq_slot[seq] * state_stride + tail_off;
    float y[PER];
    float sq = 0.0f;
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int d = tid + 128 * e;
        y[e] = 0.0f;
        if (d >= width) continue;
        const int c = base + d;
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int src = i - (taps - 1 - j);
            const float x = src >= 0
                ? gdr_slab_sum(proj + (size_t)(row - (taps - 1 - j)) * proj_stride, c, n_partials, partial_stride)
                : tail[(size_t)(taps - 1 + src) * C + c];
            acc = fmaf(fb_to_float(conv_w[(size_t)c * taps + j]), x, acc);
        }
        y[e] = gdr_silu(acc);
        sq = fmaf(y[e], y[e], sq);
    }
    float f = 1.0f;
    if (!is_v) {                                       // block-uniform
        sq = fb_block_sum(sq, red);
        f = (unit < G ? q_scale : 1.0f) / sqrtf(sq + unit_eps);
    }
    float* out = qkv + (size_t)row * C + base;
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int d = tid + 128 * e;
        if (d < width) out[d] = y[e] * f;
    }
    if (is_v && tid == 0) {
        const int h = unit - 2 * G;
        const float* pr = proj + (size_t)row * proj_stride;
        const float b = gdr_slab_sum(pr, C + h, n_partials, partial_stride);
        const float a = gdr_slab_sum(pr, C + H + h, n_partials, partial_stride);
        beta[(size_t)row * H + h] = 1.0f / (1.0f + expf(-b));
        decay[(size_t)row * H + h] = expf(-expf(fb_to_float(a_log[h])) * gdr_softplus(a + fb_to_float(dt_bias[h])));
    }
}

__global__ void gdr_conv_tail_kernel(const float* __restrict__ proj, long proj_stride, int n_partials, long partial_stride,
                                     int taps, float* __restrict__ state, long state_stride, long tail_off,
                                     const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                                     const int* __restrict__ seq_slot, int C) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int L = seq_q_len[seq], start = seq_q_start[seq];
    float* tail = state + (size_t)seq_slot[seq] * state_stride + tail_off;
    // ascending m: an entry taken from the old tail lies above the one being written
    for (int m = 0; m < taps - 1; ++m) {
        const int src = L - (taps - 1) + m;
        tail[(size_t)m * C + c] = src >= 0
            ? gdr_slab_sum(proj + (size_t)(start + src) * proj_stride, c, n_partials, partial_stride)
            : tail[(size_t)(taps - 1 + src) * C + c];
    }
}

// A 4-byte copy from global to shared memory that does not pass through registers (the thread goes on at once).
__device__ __forceinline__ void gdr_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void gdr_copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT> __device__ __forceinline__ void gdr_copies_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory");
}

// LPC lanes a column, R state values a lane (the key dimension d = lane + LPC r, dk <= LPC R), 256 / LPC columns a CTA.
template <int R, int LPC> struct GdrTile {
    static constexpr int THREADS = 256, COLS = THREADS / LPC, DKP = LPC * R;
    // tokens fetched at a time: two such stretches are in shared memory, one being worked on, one arriving
    static constexpr int CH = DKP <= 128 ? 32 : DKP <= 256 ? 16 : 8;
    static constexpr int STAGE_FLOATS = CH * (2 * DKP + COLS + 5);
    __device__ static constexpr int place(int d) { return d; }     // where dimension d of a row lies in shared memory
};

template <int R, int LPC>
__global__ void __launch_bounds__(256)
gdr_recurrent_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                     float* __restrict__ state, long state_stride, const int* __restrict__ seq_q_start,
                     const int* __restrict__ seq_q_len, const int* __restrict__ seq_slot, float* __restrict__ o,
                     int G, int H, int dk, int dv) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    using Tile = GdrTile<R, LPC>;
    constexpr int THREADS = Tile::THREADS, COLS = Tile::COLS, CH = Tile::CH, DKP = Tile::DKP;
    extern __shared__ __align__(16) float sh[];
    const int seq = blockIdx.x / H, head = blockIdx.x - seq * H;
    const int g = head / (H / G);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int li = tid % LPC, col = blockIdx.y * COLS + tid / LPC;
    const bool live = col < dv;
    const int qk = G * dk, C = 2 * qk + H * dv;
    const int start = seq_q_start[seq], L = seq_q_len[seq];
    float* S = state + (size_t)seq_slot[seq] * state_stride + ((size_t)head * dv + (live ? col : 0)) * dk;

    // a stage: q [CH][DKP], k [CH][DKP] (rows padded with zeros beyond dk), v [CH][COLS], then [CH] each: beta, decay,
    // k_t . q_t, k_t . k_t+1, k_t . q_t+1
    auto fetch = [&](int t0, float* st) {
        const int cnt = min(CH, L - t0);
        float* qs = st;
        float* ks = qs + CH * DKP;
        float* vs = ks + CH * DKP;
        float* bs = vs + CH * COLS;
        float* gs = bs + CH;
        for (int e = tid; e < cnt * DKP; e += THREADS) {
            const int t = e / DKP, d = e - t * DKP;
            const float* rowp = qkv + (size_t)(start + t0 + t) * C + (size_t)g * dk;
            const int at = t * DKP + Tile::place(d);
            if (d < dk) {
                gdr_copy4(qs + at, rowp + d);
                gdr_copy4(ks + at, rowp + qk + d);
            } else {
                qs[at] = 0.0f;
                ks[at] = 0.0f;
            }
        }
        for (int e = tid; e < cnt * COLS; e += THREADS) {
            const int t = e / COLS, c2 = blockIdx.y * COLS + (e - t * COLS);
            if (c2 < dv) gdr_copy4(vs + e, qkv + (size_t)(start + t0 + t) * C + 2 * qk + (size_t)head * dv + c2);
            else vs[e] = 0.0f;
        }
        if (tid < cnt) {
            gdr_copy4(bs + tid, beta + (size_t)(start + t0 + tid) * H + head);
            gdr_copy4(gs + tid, decay + (size_t)(start + t0 + tid) * H + head);
        }
        gdr_copies_commit();
    };

    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = li + LPC * r;
        s[r] = (live && d < dk) ? S[d] : 0.0f;
    }
    if (L > 0) fetch(0, sh);
    int buf = 0;
    for (int t0 = 0; t0 < L; t0 += CH, buf ^= 1) {
        const int cnt = min(CH, L - t0);
        float* st = sh + buf * Tile::STAGE_FLOATS;
        const bool more = t0 + CH < L;
        if (more) fetch(t0 + CH, sh + (buf ^ 1) * Tile::STAGE_FLOATS);    // (its last readers passed the barrier below)
        if (more) gdr_copies_wait<1>(); else gdr_copies_wait<0>();
        __syncthreads();
        const float* qs = st;
        const float* ks = qs + CH * DKP;
        const float* vs = ks + CH * DKP;
        const float* bs = vs + CH * COLS;
        const float* gs = bs + CH;
        float* kq = st + CH * (2 * DKP + COLS + 2);
        float* kkn = kq + CH;                          // k_t . k_t+1
        float* kqn = kkn + CH;                         // k_t . q_t+1
        for (int t = warp; t < cnt; t += THREADS / 32) {
            const bool pair = !(t & 1) && t + 1 < cnt;
            float acc = 0.0f, acc_k = 0.0f, acc_q = 0.0f;
            for (int d = lane; d < DKP; d += 32) {
                const float kd = ks[t * DKP + d];
                acc = fmaf(kd, qs[t * DKP + d], acc);
                if (pair) {
                    acc_k = fmaf(kd, ks[(t + 1) * DKP + d], acc_k);
                    acc_q = fmaf(kd, qs[(t + 1) * DKP + d], acc_q);
                }
            }
            acc = fb_warp_sum(acc);
            acc_k = fb_warp_sum(acc_k);
            acc_q = fb_warp_sum(acc_q);
            if (lane == 0) { kq[t] = acc; kkn[t] = acc_k; kqn[t] = acc_q; }
        }
        __syncthreads();
        int t = 0;
        // Two tokens at a time: all four products with the state are taken from the state before either update and
        // share one exchange between the lanes; the second token's follow from the first's correction:
        //   S_t^T k_t+1 = g_t S_t-1^T k_t+1 + u_t (k_t . k_t+1), and likewise for q_t+1;
        //   S_t+1 = g_t+1 g_t S_t-1 + g_t+1 k_t u_t^T + k_t+1 u_t+1^T.
        for (; t + 1 < cnt; t += 2) {
            const float g0 = gs[t], g1 = gs[t + 1];
            const float* k0p = ks + t * DKP + li;
            const float* q0p = qs + t * DKP + li;
            float k0[R], k1[R];
            float a0 = 0.0f, b0 = 0.0f, a1 = 0.0f, b1 = 0.0f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                k0[r] = k0p[LPC * r];
                k1[r] = k0p[DKP + LPC * r];
                a0 = fmaf(s[r], k0[r], a0);
                b0 = fmaf(s[r], q0p[LPC * r], b0);
                a1 = fmaf(s[r], k1[r], a1);
                b1 = fmaf(s[r], q0p[DKP + LPC * r], b1);
            }
#pragma unroll
            for (int off = LPC / 2; off > 0; off >>= 1) {
                a0 += __shfl_xor_sync(0xffffffffu, a0, off);
                b0 += __shfl_xor_sync(0xffffffffu, b0, off);
                a1 += __shfl_xor_sync(0xffffffffu, a1, off);
                b1 += __shfl_xor_sync(0xffffffffu, b1, off);
            }
            const float u0 = bs[t] * (vs[t * COLS + tid / LPC] - g0 * a0);
            const float a1n = fmaf(u0, kkn[t], g0 * a1);
            const float u1 = bs[t + 1] * (vs[(t + 1) * COLS + tid / LPC] - g1 * a1n);
            const float b1n = fmaf(u0, kqn[t], g0 * b1);
            const float gg = g1 * g0, gu = g1 * u0;
#pragma unroll
            for (int r = 0; r < R; ++r) s[r] = fmaf(k1[r], u1, fmaf(k0[r], gu, gg * s[r]));
            if (live && li == 0) {
                float* op = o + (size_t)(start + t0 + t) * H * dv + (size_t)head * dv + col;
                op[0] = fmaf(u0, kq[t], g0 * b0);
                op[(size_t)H * dv] = fmaf(u1, kq[t + 1], g1 * b1n);
            }
        }
        for (; t < cnt; ++t) {
            const float gt = gs[t];
            const float* kt = ks + t * DKP + li;
            const float* qt = qs + t * DKP + li;
            float kk[R];
            float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                kk[r] = kt[LPC * r];
                const float qq = qt[LPC * r];
                if (r & 1) { a1 = fmaf(s[r], kk[r], a1); b1 = fmaf(s[r], qq, b1); }
                else { a0 = fmaf(s[r], kk[r], a0); b0 = fmaf(s[r], qq, b0); }
            }
            float a = a0 + a1, b = b0 + b1;
#pragma unroll
            for (int off = LPC / 2; off > 0; off >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, off);
                b += __shfl_xor_sync(0xffffffffu, b, off);
            }
            const float u = bs[t] * (vs[t * COLS + tid / LPC] - gt * a);
#pragma unroll
            for (int r = 0; r < R; ++r) s[r] = fmaf(kk[r], u, gt * s[r]);
            if (live && li == 0)
                o[(size_t)(start + t0 + t) * H * dv + (size_t)head * dv + col] = fmaf(u, kq[t], gt * b);
        }
        __syncthreads();                               // the stage may be overwritten by the fetch after next
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = li + LPC * r;
        if (live && d < dk) S[d] = s[r];
    }
}

template <typename TW, typename T>
__global__ void __launch_bounds__(128)
gdr_out_norm_kernel(const float* __restrict__ o, const float* __restrict__ proj, long proj_stride, int n_partials,
                    long partial_stride, int gate_off, const TW* __restrict__ weight, float eps, T* __restrict__ out,
                    int n, int H, int dv) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 4 + warp;
    if (item >= (long)n * H) return;
    const int row = (int)(item / H), head = (int)(item - (long)row * H);
    const float* x = o + (size_t)row * H * dv + (size_t)head * dv;
    float s = 0.0f;
    for (int d = lane; d < dv; d += 32) s = fmaf(x[d], x[d], s);
    s = fb_warp_sum(s);
    const float inv = 1.0f / sqrtf(s / (float)dv + eps);
    const float* pr = proj + (size_t)row * proj_stride;
    for (int d = lane; d < dv; d += 32) {
        const float gate = gdr_slab_sum(pr, gate_off + head * dv + d, n_partials, partial_stride);
        out[(size_t)row * H * dv + (size_t)head * dv + d] =
            fb_from_float<T>(x[d] * inv * fb_to_float(weight[d]) * gdr_silu(gate));
    }
}

FB_API int fb_gdr_prepare(const float* proj, long long proj_stride, int n_partials, long long partial_stride,
                          const void* conv_w, int taps, const void* a_log, const void* dt_bias, int w_dtype,
                          float* state, long long state_stride, long long tail_off, const int* row_seq,
                          const int* seq_q_start, const int* seq_q_len, const int* seq_slot, int n_seqs, float* qkv,
                          float* beta, float* decay, int n, int G, int H, int dk, int dv, float q_scale,
                          float unit_eps, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && G > 0 && H > 0 && H % G == 0 && dk > 0 && dv > 0 && taps >= 1, "gated delta: bad sizes");
    const long long C = 2LL * G * dk + (long long)H * dv;
    FB_REQUIRE(proj_stride >= C + 2LL * H + (long long)H * dv, "gated delta: projection rows are too short");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    FB_REQUIRE(dk <= 1024 && dv <= 1024, "gated delta: head sizes up to 1024 (key %d, value %d)", dk, dv);
    FB_REQUIRE(2 * G + H <= 65535, "gated delta: too many heads");
    FB_DISPATCH_DTYPE(w_dtype, TW, {
        auto kernel = gdr_prepare_kernel<TW>;
        fb_launch(kernel, dim3(n, 2 * G + H), dim3(128), 0, stream, proj, (long)proj_stride, n_partials, (long)partial_stride,
                  (const TW*)conv_w, taps, (const TW*)a_log, (const TW*)dt_bias, (const float*)state, (long)state_stride,
                  (long)tail_off, row_seq, seq_q_start, seq_slot, qkv, beta, decay, G, H, dk, dv, q_scale, unit_eps);
    });
    int rc = fb_check_launch("gdr_prepare");
    if (rc || taps < 2) return rc;
    fb_launch(gdr_conv_tail_kernel, dim3(n_seqs, (unsigned)((C + 127) / 128)), dim3(128), 0, stream, proj,
              (long)proj_stride, n_partials, (long)partial_stride, taps, state, (long)state_stride, (long)tail_off,
              seq_q_start, seq_q_len, seq_slot, (int)C);
    return fb_check_launch("gdr_conv_tail");
}

template <int R, int LPC>
static int launch_gdr_recurrent(const float* qkv, const float* beta, const float* decay, float* state,
                                long state_stride, const int* seq_q_start, const int* seq_q_len, const int* seq_slot,
                                int n_seqs, float* o, int G, int H, int dk, int dv, cudaStream_t stream) {
    using Tile = GdrTile<R, LPC>;
    const size_t smem = (size_t)2 * Tile::STAGE_FLOATS * sizeof(float);
    auto kernel = gdr_recurrent_kernel<R, LPC>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    fb_launch(kernel, dim3(n_seqs * H, (dv + Tile::COLS - 1) / Tile::COLS), dim3(Tile::THREADS), smem, stream, qkv, beta,
              decay, state, state_stride, seq_q_start, seq_q_len, seq_slot, o, G, H, dk, dv);
    return fb_check_launch("gdr_recurrent");
}

FB_API int fb_gdr_recurrent(const float* qkv, const float* beta, const float* decay, float* state,
                            long long state_stride, const int* seq_q_start, const int* seq_q_len, const int* seq_slot,
                            int n_seqs, float* o, int G, int H, int dk, int dv, cudaStream_t stream) {
    FB_REQUIRE(n_seqs >= 0 && G > 0 && H > 0 && H % G == 0 && dk > 0 && dv > 0, "gated delta: bad sizes");
    FB_REQUIRE(dk <= 1024, "gated delta: key size %d is larger than 1024", dk);
    if (n_seqs == 0) return 0;
#define FB_GDR_CASE(R, LPC) return launch_gdr_recurrent<R, LPC>(qkv, beta, decay, state, (long)state_stride, seq_q_start, \
        seq_q_len, seq_slot, n_seqs, o, G, H, dk, dv, stream)
    // (sixteen lanes a column and 256 threads measured fastest for keys of 128: fewer lanes leave too few warps to
    // hide the exchange between lanes, more lanes spend their instructions on that exchange)
    if (dk <= 16) FB_GDR_CASE(1, 16);
    if (dk <= 32) FB_GDR_CASE(2, 16);
    if (dk <= 64) FB_GDR_CASE(4, 16);
    if (dk <= 128) FB_GDR_CASE(8, 16);
    if (dk <= 256) FB_GDR_CASE(16, 16);
    if (dk <= 512) FB_GDR_CASE(16, 32);
    FB_GDR_CASE(32, 32);
#undef FB_GDR_CASE
}

FB_API int fb_gdr_out_norm(const float* o, const float* proj, long long proj_stride, int n_partials,
                           long long partial_stride, int gate_off, const void* weight, int w_dtype, float eps,
                           void* out, int out_dtype, int n, int H, int dv, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && H > 0 && dv > 0, "gated delta: bad sizes");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    const long items = (long)n * H;
    FB_DISPATCH_DTYPE(w_dtype, TW, FB_DISPATCH_DTYPE(out_dtype, T,
        (fb_launch((gdr_out_norm_kernel<TW, T>), dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, o, proj,
                   (long)proj_stride, n_partials, (long)partial_stride, gate_off, (const TW*)weight, eps, (T*)out, n, H,
                   dv))));
    return fb_check_launch("gdr_out_norm");
}
