// Differential attention over the paged cache: what lies between the fused projection and the output projection.
//
// A head h has two score maps over the same values.  Queries are [tokens][H][2][kd] (map 1 then map 2 of a head),
// keys live in the cache as [page][G][slot][2*kd] (both maps of a key/value head side by side) and values as
// [page][G][slot][vd]; kd and vd are independent.  Per token and head:
//     a_m = softmax_j(scale * q_m . k_m[j]) V        over the keys j in [max(0, p - W + 1), p]   (W = 0: all of [0, p])
//     o   = a_1 - lambda * a_2
//     o  <- o / sqrt(mean(o^2) + eps) * out_scale * gate[token][h]            (gate optional)
// Scores, softmax weights, the weighted sums, the difference and the norm are float32 whatever the storage type.
//
//   fb_qkv_bias_cache_write   adds the split-K shares of the fused projection and the biases, writes q, puts k and v
//                             into their pages, and turns the gate columns into sigmoid(g)
//   fb_diff_attention_simt    one warp per (token, head), float32 math on the CUDA cores: the attention of the 32-bit
//                             mode, of sizes the tensor-core arrangements do not take, and their reference
#include "common.cuh"

// ---------------------------------------------------------------------------
// Fused projection -> q, cache, gate.
// A row of `proj` holds [q: nh*qd | k: nkv*qd | v: nkv*vd | g: n_gate] (qd = both maps of a head = 2*kd for the
// differential mixer), as `n_partials` float32 slabs `partial_stride` elements apart.  `bias` (optional) covers the
// q, k and v columns.  grid (tokens, ceil(columns / 256)).
// ---------------------------------------------------------------------------
template <typename TB, typename T>
__global__ void qkv_bias_cache_write_kernel(const float* __restrict__ proj, long proj_stride, int n_partials,
                                            long partial_stride, const TB* __restrict__ bias, T* __restrict__ q_out,
                                            long q_out_stride, float* __restrict__ gate_out,
                                            const int* __restrict__ positions, const int* __restrict__ row_seq,
                                            const int* __restrict__ block_table, int table_stride,
                                            const int* __restrict__ table_base, T* __restrict__ k_pool,
                                            T* __restrict__ v_pool, int page_size, int n_pages, int nh, int nkv,
                                            int qd, int vd, int n_gate, int write_kv, int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int t = blockIdx.x;
    const int qw = nh * qd, kw = nkv * qd, vw = nkv * vd;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= qw + kw + vw + n_gate) return;
    const float* src = proj + (size_t)t * proj_stride + c;
    float val = 0.0f;
    for (int p = 0; p < n_partials; ++p) val += src[(size_t)p * partial_stride];
    if (c >= qw + kw + vw) {                                   // gate columns: no bias
        gate_out[(size_t)t * n_gate + (c - qw - kw - vw)] = 1.0f / (1.0f + expf(-val));
        return;
    }
    if (bias) val += fb_to_float(bias[c]);
    if (c < qw) {
        q_out[(size_t)t * q_out_stride + c] = fb_from_float<T>(val);
        return;
    }
    if (!write_kv) return;
    const int pos = positions[t], seq = row_seq[t];
    const int entry = pos / page_size - (table_base ? table_base[seq] : 0);
    const int page = (entry >= 0 && entry < table_stride) ? block_table[(size_t)seq * table_stride + entry] : -1;
    if (page < 0 || page >= n_pages) {
        atomicOr(status, FB_STATUS_BAD_PAGE);
        return;
    }
    const int slot = pos % page_size;
    if (c < qw + kw) {
        const int j = c - qw, h = j / qd, d = j - h * qd;
        k_pool[(((size_t)page * nkv + h) * page_size + slot) * qd + d] = fb_from_float<T>(val);
    } else {
        const int j = c - qw - kw, h = j / vd, d = j - h * vd;
        v_pool[(((size_t)page * nkv + h) * page_size + slot) * vd + d] = fb_from_float<T>(val);
    }
}

// The same four columns at a time (head sizes multiples of 4, aligned rows): grid (tokens, ceil(items / 256)), an
// item being four consecutive q, k or v columns; the gate columns follow as single items.
template <typename T> struct Row4 {};
template <> struct Row4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Row4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename TB, typename T>
__global__ void __launch_bounds__(256)
qkv_bias_cache_write_vec_kernel(const float* __restrict__ proj, long proj_stride, int n_partials, long partial_stride,
                                const TB* __restrict__ bias, T* __restrict__ q_out, long q_out_stride,
                                float* __restrict__ gate_out, const int* __restrict__ positions,
                                const int* __restrict__ row_seq, const int* __restrict__ block_table, int table_stride,
                                const int* __restrict__ table_base, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                int page_size, int n_pages, int nh, int nkv, int qd, int vd, int n_gate, int write_kv,
                                int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int t = blockIdx.x;
    const int qw = nh * qd, kw = nkv * qd, vw = nkv * vd;
    const int vec_items = (qw + kw + vw) >> 2;
    const int item = blockIdx.y * blockDim.x + threadIdx.x;
    if (item >= vec_items + n_gate) return;
    if (item >= vec_items) {                                   // a gate column
        const int c = qw + kw + vw + (item - vec_items);
        const float* src = proj + (size_t)t * proj_stride + c;
        float val = 0.0f;
        for (int p = 0; p < n_partials; ++p) val += src[(size_t)p * partial_stride];
        gate_out[(size_t)t * n_gate + (item - vec_items)] = 1.0f / (1.0f + expf(-val));
        return;
    }
    const int c = item << 2;
    if (c >= qw && !write_kv) return;
    const float* src = proj + (size_t)t * proj_stride + c;
    float4 val = Row4<float>::load(src);
    for (int p = 1; p < n_partials; ++p) {
        const float4 e = Row4<float>::load(src + (size_t)p * partial_stride);
        val.x += e.x; val.y += e.y; val.z += e.z; val.w += e.w;
    }
    if (bias) {
        const float4 b = Row4<TB>::load(bias + c);
        val.x += b.x; val.y += b.y; val.z += b.z; val.w += b.w;
    }
    if (c < qw) {
        Row4<T>::store(q_out + (size_t)t * q_out_stride + c, val);
        return;
    }
    const int pos = positions[t], seq = row_seq[t];
    const int entry = pos / page_size - (table_base ? table_base[seq] : 0);
    const int page = (entry >= 0 && entry < table_stride) ? block_table[(size_t)seq * table_stride + entry] : -1;
    if (page < 0 || page >= n_pages) {
        atomicOr(status, FB_STATUS_BAD_PAGE);
        return;
    }
    const int slot = pos % page_size;
    if (c < qw + kw) {
        const int j = c - qw, h = j / qd, d = j - h * qd;
        Row4<T>::store(k_pool + (((size_t)page * nkv + h) * page_size + slot) * qd + d, val);
    } else {
        const int j = c - qw - kw, h = j / vd, d = j - h * vd;
        Row4<T>::store(v_pool + (((size_t)page * nkv + h) * page_size + slot) * vd + d, val);
    }
}

FB_API int fb_qkv_bias_cache_write(const float* proj, long long proj_stride, int n_partials, long long partial_stride,
                                   const void* bias, int bias_dtype, void* q_out, long long q_out_stride,
                                   int out_dtype, float* gate_out, const int* positions, const int* row_seq,
                                   const int* block_table, int table_stride, const int* table_base, void* k_pool,
                                   void* v_pool, int page_size, int n_pages, int n, int nh, int nkv, int qd, int vd,
                                   int n_gate, int write_kv, int* status, cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && nh > 0 && nkv > 0 && qd > 0 && vd > 0 && n_gate >= 0, "qkv_bias_cache_write: bad sizes");
    FB_REQUIRE(n_gate == 0 || gate_out, "qkv_bias_cache_write: gate columns without a place for them");
    FB_REQUIRE(!write_kv || (page_size > 0 && n_pages > 0 && k_pool && v_pool && block_table && positions && row_seq),
               "qkv_bias_cache_write: cache arguments missing");
    if (n == 0) return 0;
    if (n_partials < 1) n_partials = 1;
    const int cols = nh * qd + nkv * qd + nkv * vd + n_gate;
    FB_REQUIRE(proj_stride >= cols, "qkv_bias_cache_write: rows of %lld for %d columns", proj_stride, cols);
    if (!bias) bias_dtype = FB_F32;
    const bool vec = qd % 4 == 0 && vd % 4 == 0 && proj_stride % 4 == 0 && partial_stride % 4 == 0 &&
                     q_out_stride % 4 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)bias % 16 == 0 &&
                     (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0;
    if (vec) {
        const int items = (cols - n_gate) / 4 + n_gate;
        FB_DISPATCH_DTYPE(bias_dtype, TB, FB_DISPATCH_DTYPE(out_dtype, T,
            (fb_launch((qkv_bias_cache_write_vec_kernel<TB, T>), dim3(n, (items + 255) / 256), 256, 0, stream, proj,
                       (long)proj_stride, n_partials, (long)partial_stride, (const TB*)bias, (T*)q_out,
                       (long)q_out_stride, gate_out, positions, row_seq, block_table, table_stride, table_base,
                       (T*)k_pool, (T*)v_pool, page_size, n_pages, nh, nkv, qd, vd, n_gate, write_kv, status))));
        return fb_check_launch("qkv_bias_cache_write");
    }
    FB_DISPATCH_DTYPE(bias_dtype, TB, FB_DISPATCH_DTYPE(out_dtype, T,
        (fb_launch((qkv_bias_cache_write_kernel<TB, T>), dim3(n, (cols + 255) / 256), 256, 0, stream, proj,
                   (long)proj_stride, n_partials, (long)partial_stride, (const TB*)bias, (T*)q_out, (long)q_out_stride,
                   gate_out, positions, row_seq, block_table, table_stride, table_base, (T*)k_pool, (T*)v_pool,
                   page_size, n_pages, nh, nkv, qd, vd, n_gate, write_kv, status))));
    return fb_check_launch("qkv_bias_cache_write");
}

// ---------------------------------------------------------------------------
// The float32-math kernel.  A warp walks the visible keys 32 at a time: each lane scores one key for both maps,
// the warp agrees on each map's running maximum, and the lanes then split the value dimensions.
// ---------------------------------------------------------------------------
template <typename T, int NDR>   // NDR = ceil(vd / 32) accumulator registers per lane and map
__global__ void __launch_bounds__(128)
diff_attention_simt_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                           const float* __restrict__ gate, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                           int page_size, int n_pages, const int* __restrict__ block_table, int table_stride,
                           const int* __restrict__ table_base, const int* __restrict__ positions,
                           const int* __restrict__ row_seq, int n, int nh, int nkv, int kd, int vd, int window,
                           float scale, float lambda, float eps, float out_scale, int* status) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    extern __shared__ float q_sh[];                    // [4 warps][2 * kd]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 4 + warp;
    const bool active = item < (long)n * nh;
    const int row = active ? (int)(item / nh) : 0;
    const int head = active ? (int)(item - (long)row * nh) : 0;
    const int kvh = head / (nh / nkv);
    const int qd = 2 * kd;
    float* qs = q_sh + warp * qd;
    if (active) {
        const T* qp = q + (size_t)row * q_stride + (size_t)head * qd;
        for (int d = lane; d < qd; d += 32) qs[d] = fb_to_float(qp[d]);
    }
    __syncwarp();
    if (!active) return;

    const int p = positions[row];
    const int t0 = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int* table = block_table + (size_t)row_seq[row] * table_stride;
    const int base_page = table_base ? table_base[row_seq[row]] : 0;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float acc[2][NDR];
#pragma unroll
    for (int r = 0; r < NDR; ++r) acc[0][r] = acc[1][r] = 0.0f;

    for (int base = t0; base <= p; base += 32) {
        const int t = base + lane;
        float s[2] = {-INFINITY, -INFINITY};
        int my_page = -1;
        if (t <= p) {
            const int entry = t / page_size - base_page;
            my_page = (entry >= 0 && entry < table_stride) ? table[entry] : -1;
            if (my_page < 0 || my_page >= n_pages) {
                atomicOr(status, FB_STATUS_BAD_PAGE);
                my_page = -1;
            } else {
                const T* kr = k_pool + (((size_t)my_page * nkv + kvh) * page_size + (t % page_size)) * qd;
                float d0 = 0.0f, d1 = 0.0f;
                for (int d = 0; d < kd; ++d) {
                    d0 = fmaf(qs[d], fb_to_float(kr[d]), d0);
                    d1 = fmaf(qs[kd + d], fb_to_float(kr[kd + d]), d1);
                }
                s[0] = d0 * scale;
                s[1] = d1 * scale;
            }
        }
        float pr[2];
#pragma unroll
        for (int mp = 0; mp < 2; ++mp) {
            const float tile_max = fb_warp_max(s[mp]);
            const float m_new = fmaxf(m[mp], tile_max);
            const float corr = (m[mp] == -INFINITY) ? 0.0f : expf(m[mp] - m_new);
            pr[mp] = (s[mp] == -INFINITY) ? 0.0f : expf(s[mp] - m_new);
            l[mp] = l[mp] * corr + fb_warp_sum(pr[mp]);
#pragma unroll
            for (int r = 0; r < NDR; ++r) acc[mp][r] *= corr;
            m[mp] = m_new;
        }
        const int count = min(32, p - base + 1);
        for (int j = 0; j < count; ++j) {
            const float p0 = __shfl_sync(0xffffffffu, pr[0], j);
            const float p1 = __shfl_sync(0xffffffffu, pr[1], j);
            const int page_j = __shfl_sync(0xffffffffu, my_page, j);
            if (page_j < 0) continue;
            const int tj = base + j;
            const T* vr = v_pool + (((size_t)page_j * nkv + kvh) * page_size + (tj % page_size)) * vd;
#pragma unroll
            for (int r = 0; r < NDR; ++r) {
                const int d = lane + 32 * r;
                if (d < vd) {
                    const float v = fb_to_float(vr[d]);
                    acc[0][r] = fmaf(p0, v, acc[0][r]);
                    acc[1][r] = fmaf(p1, v, acc[1][r]);
                }
            }
        }
    }
    const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
    float o[NDR], ss = 0.0f;
#pragma unroll
    for (int r = 0; r < NDR; ++r) {
        const int d = lane + 32 * r;
        o[r] = d < vd ? acc[0][r] * inv0 - lambda * (acc[1][r] * inv1) : 0.0f;
        ss += o[r] * o[r];
    }
    ss = fb_warp_sum(ss);
    const float f = out_scale * (gate ? gate[(size_t)row * nh + head] : 1.0f) / sqrtf(ss / (float)vd + eps);
    T* op = out + (size_t)row * out_stride + (size_t)head * vd;
#pragma unroll
    for (int r = 0; r < NDR; ++r) {
        const int d = lane + 32 * r;
        if (d < vd) op[d] = fb_from_float<T>(o[r] * f);
    }
}

template <typename T, int NDR>
static int launch_diff_simt(const void* q, long q_stride, void* out, long out_stride, const float* gate,
                            const void* k_pool, const void* v_pool, int page_size, int n_pages, const int* block_table,
                            int table_stride, const int* table_base, const int* positions, const int* row_seq, int n,
                            int nh, int nkv, int kd, int vd, int window, float scale, float lambda, float eps,
                            float out_scale, int* status, cudaStream_t stream) {
    const long items = (long)n * nh;
    fb_launch((diff_attention_simt_kernel<T, NDR>), (unsigned)((items + 3) / 4), 128, 8 * kd * sizeof(float), stream,
              (const T*)q, q_stride, (T*)out, out_stride, gate, (const T*)k_pool, (const T*)v_pool, page_size, n_pages,
              block_table, table_stride, table_base, positions, row_seq, n, nh, nkv, kd, vd, window, scale, lambda,
              eps, out_scale, status);
    return fb_check_launch("diff_attention_simt");
}

FB_API int fb_diff_attention_simt(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                                  const float* gate, const void* k_pool, const void* v_pool, int page_size,
                                  int n_pages, const int* block_table, int table_stride, const int* table_base,
                                  const int* positions, const int* row_seq, int n, int nh, int nkv, int kd, int vd,
                                  int window, float scale, float lambda, float eps, float out_scale, int* status,
                                  cudaStream_t stream) {
    FB_REQUIRE(n >= 0 && nh > 0 && nkv > 0 && kd > 0 && vd > 0, "diff attention: bad sizes");
    FB_REQUIRE(nh % nkv == 0, "diff attention: %d query heads are not a multiple of %d key/value heads", nh, nkv);
    FB_REQUIRE(vd <= 512 && kd <= 1024, "diff attention: head sizes %d / %d are too large", kd, vd);
    FB_REQUIRE(page_size > 0 && n_pages > 0 && window >= 0 && eps > 0.0f, "diff attention: bad cache geometry or eps");
    if (n == 0) return 0;
#define FB_DIFF_CASE(NDR)                                                                                          \
    FB_DISPATCH_DTYPE(dtype, T, return (launch_diff_simt<T, NDR>(q, (long)q_stride, out, (long)out_stride, gate,   \
        k_pool, v_pool, page_size, n_pages, block_table, table_stride, table_base, positions, row_seq, n, nh, nkv, \
        kd, vd, window, scale, lambda, eps, out_scale, status, stream)))
    if (vd <= 32) { FB_DIFF_CASE(1); }
    else if (vd <= 64) { FB_DIFF_CASE(2); }
    else if (vd <= 128) { FB_DIFF_CASE(4); }
    else if (vd <= 256) { FB_DIFF_CASE(8); }
    else { FB_DIFF_CASE(16); }
#undef FB_DIFF_CASE
    return 0;
}
