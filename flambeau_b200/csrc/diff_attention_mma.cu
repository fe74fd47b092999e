// Differential attention on the tensor cores (mma.sync, bfloat16 operands, float32 accumulation) over the paged cache.
// The math is that of diff_attention.cu; q, k, v arrive rounded to bfloat16, everything after them is float32.
//
// Rows.  The rows of a sequence are (token, query head of one key/value head) pairs, token-major: row R of
// (sequence, key/value head g) is token R / HG, head g * HG + R % HG (HG = query heads per key/value head).  All
// rows of a CTA share every K/V tile it fetches, so grouped heads cost no second read of the cache.  A warp owns 16
// rows of ONE map; the warps of map 1 and the warps of map 2 of the same rows sit in one CTA and meet at the end.
//
// Two arrangements of one kernel:
//   portions  (rows of the sequence > short_rows): a CTA owns 64 rows (4 warps per map), walks the 64-key tiles its
//             rows can see, every warp scoring the whole tile for its 16 rows (32 keys at a time), and ends with the epilogue
//             (a1 - lambda a2, head norm, gate) through shared memory.
//   split     (rows <= 16: decoded tokens and portions of a few tokens): a CTA owns the 16 rows of (sequence, g) and
//             a stretch of the key tiles; its 4 warps per map take 16 keys of each tile each and never meet: every
//             warp leaves a partial (running maximum, sum, unnormalised output) per row, and
//             diff_attention_combine_kernel merges the partials of all stretches and warps and runs the epilogue.
//
// The softmax weights stay float32 into the second product: a weight p is fed as two bfloat16 terms, p_hi = bf16(p)
// and p_lo = bf16(p - p_hi), so P V carries 16 bits of p's mantissa instead of 8 (two MMAs where a kernel that
// rounds P issues one).  K/V tiles arrive by 16-byte cp.async copies through three stages where shared memory has
// room (two tiles in flight while one is used; one barrier a tile), else two; rows outside the visible range or
// without a page are zero-filled.  Tiles that all rows of a warp see whole skip the mask.
#include "attention_common.cuh"

namespace {

using namespace fb_attn;

struct DiffArgs {
    const __nv_bfloat16* q; long q_stride;
    __nv_bfloat16* out; long out_stride;
    const float* gate;                   // [rows of the step][nh], or nullptr
    const __nv_bfloat16* k_pool; const __nv_bfloat16* v_pool;
    int page_size, n_pages;
    int page_shift;                      // log2(page_size) where it is a power of two, else -1
    const int* block_table; int table_stride; const int* table_base;
    const int* seq_q_start; const int* seq_q_len; const int* seq_pos_start;
    int n_seqs, nh, nkv, kd, vd, window;
    float scale_log2e, lambda, eps, out_scale;
    int short_rows;                      // sequences with q_len * HG <= short_rows run in the split arrangement
    int n_splits;                        // split arrangement: CTAs per (sequence, key/value head)
    int n_stages;                        // K/V tiles in shared memory (2 or 3)
    float* part_o; float* part_ml;       // partials: [slot][sequence][g][16 rows][2 maps] x vd, and x 2 (maximum, sum)
    int* status;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_to(uint32_t dst, const void* src) {          // dst: a shared-memory address
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void zero16_at(uint32_t dst) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ldmatrix from a 32-bit shared-memory address (base + byte offset), so that the address is one integer add
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ size_t part_index(const DiffArgs& a, int slot, int seq, int g, int row, int map) {
    return ((((size_t)slot * a.n_seqs + seq) * a.nkv + g) * 16 + row) * 2 + map;
}

// Portions: a warp takes a tile's 64 keys in two halves of 32 and fetches its Q fragments from shared memory as it
// goes, so that (up to value sizes of 128) a thread stays within 128 registers and two CTAs share a multiprocessor:
// with one, its eight warps leave the tensor pipe idle two cycles in three while they wait on each other's results.
// EXACT: the key size is KSTEPS * 16 and the value size VTILES * 8, known to the compiler: strides and offsets into
// shared memory are then constants and the guards of the size loops fall away (the common sizes are built that way;
// every other multiple of 16 runs the same code with the sizes as arguments).
template <int KSTEPS, int VTILES, bool SPLIT, bool EXACT>
__global__ void __launch_bounds__(256, VTILES <= 16 ? 2 : 1)
diff_attention_mma_kernel(const DiffArgs a) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    constexpr int HALVES = SPLIT ? 1 : 2;
    constexpr int NT = SPLIT ? 2 : 4;              // 8-key n-tiles that one warp scores at a time
    constexpr int QROWS = SPLIT ? 16 : 64;
    const int seq = blockIdx.z, g = blockIdx.y;
    const int HG = a.nh / a.nkv;
    const int q_len = a.seq_q_len[seq];
    const int rows_total = q_len * HG;
    if ((rows_total <= a.short_rows) != SPLIT) return;
    const int R0 = SPLIT ? 0 : (gridDim.x - 1 - blockIdx.x) * 64;   // the tiles that see the most keys start first
    if (R0 >= rows_total) return;
    const int R1 = min(R0 + QROWS, rows_total) - 1;
    const int q_start = a.seq_q_start[seq], pos_start = a.seq_pos_start[seq];
    const int kd = EXACT ? KSTEPS * 16 : a.kd, vd = EXACT ? VTILES * 8 : a.vd, W = a.window;
    const int p_first = pos_start + R0 / HG, p_last = pos_start + R1 / HG;
    const int t_lo = (W > 0 && p_first - W + 1 > 0) ? p_first - W + 1 : 0, t_hi = p_last;
    int tile_first = t_lo / KT, tile_last = t_hi / KT;
    if (SPLIT) {
        const int n_tiles = tile_last - tile_first + 1;
        const int per = (n_tiles + a.n_splits - 1) / a.n_splits;
        tile_first += blockIdx.x * per;
        tile_last = min(tile_first + per - 1, tile_last);
    }

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int map = warp >> 2;
    const int row_tile = SPLIT ? 0 : (warp & 3);
    const int koff = SPLIT ? 16 * (warp & 3) : 0;   // the warp's keys within a tile

    // ---- shared memory ----
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int KDP = kd + 8, KP = 2 * kd + 8, VP = vd + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [2 maps][QROWS][KDP]
    const int NS = a.n_stages;
    __nv_bfloat16* Ks = Qs + 2 * QROWS * KDP;                              // [stages][64][KP]
    __nv_bfloat16* Vs = Ks + (size_t)NS * KT * KP;                         // [stages][64][VP]

    // ---- Q: rows of both maps, 16 bytes at a time; rows past the end are zero ----
    {
        const int chunks = kd / 8;                                         // per row and map
        for (int c = tid; c < 2 * QROWS * chunks; c += 256) {
            const int ch = c % chunks, r = (c / chunks) % QROWS, mp = c / (chunks * QROWS);
            const int R = R0 + r;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (R < rows_total) {
                const int tok = q_start + R / HG, h = g * HG + R % HG;
                val = *reinterpret_cast<const uint4*>(a.q + (size_t)tok * a.q_stride + ((size_t)h * 2 + mp) * kd + ch * 8);
            }
            *reinterpret_cast<uint4*>(Qs + ((size_t)mp * QROWS + r) * KDP + ch * 8) = val;
        }
    }

    // ---- the tile loader: 4 threads per key row ----
    const int* table = a.block_table + (size_t)seq * a.table_stride;
    const int base_page = a.table_base ? a.table_base[seq] : 0;
    const uint32_t ks_base = smem_addr(Ks), vs_base = smem_addr(Vs);
    auto load_tile = [&](int stage, int kt) {
        const int r = tid >> 2, sub = tid & 3;
        const int t = kt * KT + r;
        bool ok = t >= t_lo && t <= t_hi;
        size_t cache_row = 0;
        if (ok) {
            const int lp = a.page_shift >= 0 ? t >> a.page_shift : t / a.page_size;
            const int slot = a.page_shift >= 0 ? t & (a.page_size - 1) : t - lp * a.page_size;
            const int e = lp - base_page;
            const int page = (e >= 0 && e < a.table_stride) ? table[e] : -1;
            if (page < 0 || page >= a.n_pages) {
                atomicOr(a.status, FB_STATUS_BAD_PAGE);
                ok = false;
            } else {
                cache_row = ((size_t)page * a.nkv + g) * a.page_size + slot;
            }
        }
        uint32_t kdst = ks_base + 2u * (uint32_t)((stage * KT + r) * KP + sub * 8);
        uint32_t vdst = vs_base + 2u * (uint32_t)((stage * KT + r) * VP + sub * 8);
        if (ok) {
            const __nv_bfloat16* ksrc = a.k_pool + cache_row * (2 * kd) + sub * 8;
            const __nv_bfloat16* vsrc = a.v_pool + cache_row * vd + sub * 8;
#pragma unroll 4
            for (int ch = sub; ch < kd / 4; ch += 4, kdst += 64, ksrc += 32) cp_async16_to(kdst, ksrc);
#pragma unroll 4
            for (int ch = sub; ch < vd / 8; ch += 4, vdst += 64, vsrc += 32) cp_async16_to(vdst, vsrc);
        } else {
            for (int ch = sub; ch < kd / 4; ch += 4, kdst += 64) zero16_at(kdst);
            for (int ch = sub; ch < vd / 8; ch += 4, vdst += 64) zero16_at(vdst);
        }
    };

    // one copy group per tile, in tile order, also where there is no tile left (an empty group): the wait below
    // can then always name the tile it needs by how many groups may still be pending
    for (int s = 0; s < NS - 1; ++s) {
        if (tile_first + s <= tile_last) load_tile(s, tile_first + s);
        cp_async_commit();
    }
    __syncthreads();                                                       // Q is in shared memory

    // ---- this thread's two rows (lane / 4 and lane / 4 + 8 of the warp's 16) ----
    int row_p[2], row_lo[2];
    bool row_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int R = R0 + row_tile * 16 + (lane >> 2) + 8 * i;
        row_ok[i] = R < rows_total;
        row_p[i] = pos_start + (row_ok[i] ? R : 0) / HG;
        row_lo[i] = (W > 0 && row_p[i] - W + 1 > 0) ? row_p[i] - W + 1 : 0;
    }

    // byte addresses in shared memory of what this lane hands to ldmatrix: its row of Q, of a K tile (row = key,
    // plain) and of a V tile (row = key, transposed), each at the lane's 8-column block
    const uint32_t q_frag = smem_addr(Qs) + 2u * (uint32_t)((map * QROWS + row_tile * 16 + (lane & 15)) * KDP + (lane >> 4) * 8);
    const uint32_t k_lane = smem_addr(Ks) + 2u * (uint32_t)(((lane >> 4) * 8 + (lane & 7)) * KP + map * kd + ((lane >> 3) & 1) * 8);
    const uint32_t v_lane = smem_addr(Vs) + 2u * (uint32_t)((((lane >> 3) & 1) * 8 + (lane & 7)) * VP + (lane >> 4) * 8);
    uint32_t qf[SPLIT ? KSTEPS : 1][4];            // the split arrangement keeps its Q fragments in registers
    if (SPLIT) {
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
            if (ks * 16 < kd) ldsm_x4(qf[SPLIT ? ks : 0], q_frag + ks * 32);
    }

    float o[VTILES][4];
#pragma unroll
    for (int vt = 0; vt < VTILES; ++vt) o[vt][0] = o[vt][1] = o[vt][2] = o[vt][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    // the warp's rows see every key of a tile when the tile lies between the last row's window start and the first
    // row's position: such tiles need no mask
    const int warp_R0 = R0 + row_tile * 16;
    const bool warp_full = warp_R0 + 15 < rows_total;
    const int warp_p_min = pos_start + warp_R0 / HG;
    const int warp_lo_max = W > 0 ? max(0, pos_start + min(warp_R0 + 15, rows_total - 1) / HG - W + 1) : 0;

    // the stage of the tile in use and the stage to refill (the one tile kt-1 used), and their byte offsets, kept
    // as running values: NS is an argument, and a division per tile and thread is not free
    int stage = 0, refill = NS - 1;
    const uint32_t k_stage_bytes = 2u * (uint32_t)(KT * KP), v_stage_bytes = 2u * (uint32_t)(KT * VP);
    uint32_t k_tile = k_lane, v_tile = v_lane;
    for (int kt = tile_first; kt <= tile_last; ++kt) {
        if (NS == 3) cp_async_wait<1>(); else cp_async_wait<0>();          // tile kt has landed ...
        __syncthreads();                                                   // ... for all threads, and tile kt-1 is done with
        if (kt + NS - 1 <= tile_last) load_tile(refill, kt + NS - 1);
        cp_async_commit();

#pragma unroll 1
        for (int hf = 0; hf < HALVES; ++hf) {
        const int koh = koff + hf * (NT * 8);              // the keys of the tile this pass takes

        // S = Q K^T for the warp's rows, map and keys
        float s[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            if (ks * 16 < kd) {
                if (!SPLIT) ldsm_x4(qf[0], q_frag + ks * 32);
                const uint32_t (&qa)[4] = qf[SPLIT ? ks : 0];
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    uint32_t kb[4];
                    ldsm_x4(kb, k_tile + 2u * (uint32_t)((koh + np * 16) * KP + ks * 16));
                    mma_bf16(s[2 * np], qa, kb[0], kb[1]);
                    mma_bf16(s[2 * np + 1], qa, kb[2], kb[3]);
                }
            }
        }
        // scale (to base-2 units), mask, row maxima
        float tmax[2] = {-INFINITY, -INFINITY};
        const int key0 = kt * KT + koh;
        // (scores stay as the product left them; the scale, positive, enters with the exponent below)
        if (warp_full && key0 + NT * 8 - 1 <= warp_p_min && key0 >= warp_lo_max) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) tmax[e >> 1] = fmaxf(tmax[e >> 1], s[nt][e]);
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int t = key0 + nt * 8 + 2 * (lane & 3) + (e & 1);
                    const bool visible = row_ok[i] && t <= row_p[i] && t >= row_lo[i];
                    s[nt][e] = visible ? s[nt][e] : -INFINITY;
                    tmax[i] = fmaxf(tmax[i], s[nt][e]);
                }
            }
        }
        // m is kept in base-2 units (score * scale * log2 e)
        float corr[2], m_use[2];
        bool grew = false;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
            const float m_new = fmaxf(m[i], tmax[i] * a.scale_log2e);
            m_use[i] = m_new == -INFINITY ? 0.0f : m_new;
            grew = grew || m_new != m[i];
            corr[i] = exp2f(m[i] - m_use[i]);               // 0 while nothing has been seen
            m[i] = m_new;
        }
        if (__any_sync(0xffffffffu, grew)) {               // once the maxima have settled nothing is rescaled
            l[0] *= corr[0];
            l[1] *= corr[1];
#pragma unroll
            for (int vt = 0; vt < VTILES; ++vt) {
                o[vt][0] *= corr[0]; o[vt][1] *= corr[0];
                o[vt][2] *= corr[1]; o[vt][3] *= corr[1];
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = exp2f(fmaf(s[nt][e], a.scale_log2e, -m_use[e >> 1]));
                s[nt][e] = p;
                l[e >> 1] += p;
            }
        }
        // O += P V, P as p_hi + p_lo
#pragma unroll
        for (int kk = 0; kk < NT / 2; ++kk) {
            uint32_t ah[4], al[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p0 = s[2 * kk + (j >> 1)][(j & 1) * 2], p1 = s[2 * kk + (j >> 1)][(j & 1) * 2 + 1];
                ah[j] = pack_bf16(p0, p1);                 // p0 in the low half, p1 in the high half
                al[j] = pack_bf16(p0 - __uint_as_float(ah[j] << 16), p1 - __uint_as_float(ah[j] & 0xffff0000u));
            }
#pragma unroll
            for (int vp = 0; vp < VTILES / 2; ++vp) {
                if (vp * 16 < vd) {
                    uint32_t vb[4];
                    ldsm_x4_trans(vb, v_tile + 2u * (uint32_t)((koh + kk * 16) * VP + vp * 16));
                    mma_bf16(o[2 * vp], ah, vb[0], vb[1]);
                    mma_bf16(o[2 * vp], al, vb[0], vb[1]);
                    mma_bf16(o[2 * vp + 1], ah, vb[2], vb[3]);
                    mma_bf16(o[2 * vp + 1], al, vb[2], vb[3]);
                }
            }
        }
        }                                                  // the tile's next half
        refill = stage;
        if (++stage == NS) { stage = 0; k_tile = k_lane; v_tile = v_lane; }
        else { k_tile += k_stage_bytes; v_tile += v_stage_bytes; }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }

    if (SPLIT) {
        // ---- leave the warp's partial for the combining kernel ----
        const int slot = blockIdx.x * 4 + (warp & 3);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = (lane >> 2) + 8 * i;
            if (!row_ok[i]) continue;
            const size_t at = part_index(a, slot, seq, g, r, map);
            if ((lane & 3) == 0) {
                a.part_ml[2 * at] = m[i];
                a.part_ml[2 * at + 1] = l[i];
            }
            float* po = a.part_o + at * vd;
#pragma unroll
            for (int vt = 0; vt < VTILES; ++vt)
                if (vt * 8 < vd)
                    *reinterpret_cast<float2*>(po + vt * 8 + 2 * (lane & 3)) = make_float2(o[vt][2 * i], o[vt][2 * i + 1]);
        }
        return;
    }

    // ---- epilogue of a portion: map 2 hands a2 = O2 / l2 over, map 1 forms the head's output ----
    __syncthreads();                                       // every warp is done with the last tile
    float* X = reinterpret_cast<float*>(Vs);               // [64 rows][vd]; the tiles are no longer needed
    const float inv[2] = {l[0] > 0.0f ? 1.0f / l[0] : 0.0f, l[1] > 0.0f ? 1.0f / l[1] : 0.0f};
    if (map == 1) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float* xr = X + (size_t)(row_tile * 16 + (lane >> 2) + 8 * i) * vd;
#pragma unroll
            for (int vt = 0; vt < VTILES; ++vt)
                if (vt * 8 < vd)
                    *reinterpret_cast<float2*>(xr + vt * 8 + 2 * (lane & 3)) =
                        make_float2(o[vt][2 * i] * inv[i], o[vt][2 * i + 1] * inv[i]);
        }
    }
    __syncthreads();
    if (map == 0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int R = R0 + row_tile * 16 + (lane >> 2) + 8 * i;
            const float* xr = X + (size_t)(row_tile * 16 + (lane >> 2) + 8 * i) * vd;
            float ss = 0.0f;
#pragma unroll
            for (int vt = 0; vt < VTILES; ++vt) {
                if (vt * 8 < vd) {
                    const float2 a2 = *reinterpret_cast<const float2*>(xr + vt * 8 + 2 * (lane & 3));
                    o[vt][2 * i] = o[vt][2 * i] * inv[i] - a.lambda * a2.x;
                    o[vt][2 * i + 1] = o[vt][2 * i + 1] * inv[i] - a.lambda * a2.y;
                    ss += o[vt][2 * i] * o[vt][2 * i] + o[vt][2 * i + 1] * o[vt][2 * i + 1];
                }
            }
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            if (!row_ok[i]) continue;
            const int tok = q_start + R / HG, h = g * HG + R % HG;
            const float f = a.out_scale * (a.gate ? a.gate[(size_t)tok * a.nh + h] : 1.0f) / sqrtf(ss / (float)vd + a.eps);
            __nv_bfloat16* op = a.out + (size_t)tok * a.out_stride + (size_t)h * vd;
#pragma unroll
            for (int vt = 0; vt < VTILES; ++vt)
                if (vt * 8 < vd)
                    *reinterpret_cast<uint32_t*>(op + vt * 8 + 2 * (lane & 3)) = pack_bf16(o[vt][2 * i] * f, o[vt][2 * i + 1] * f);
        }
    }
}

// One warp per (sequence, key/value head, row) of the split arrangement: merges the partials of all slots (at most
// 32: lane s holds slot s's maximum and sum) for both maps and runs the epilogue.  NDR = ceil(vd / 32) values per
// lane.  The partial outputs are fetched eight slots at a time, all loads issued before the first use.
template <int NDR>
__global__ void __launch_bounds__(128)
diff_attention_combine_kernel(const DiffArgs a, int n_slots) {
    fb_pdl_launch_dependents();
    fb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 4 + warp;
    if (item >= (long)a.n_seqs * a.nkv * 16) return;
    const int r = (int)(item % 16), g = (int)((item / 16) % a.nkv), seq = (int)(item / (16 * a.nkv));
    const int HG = a.nh / a.nkv;
    const int rows_total = a.seq_q_len[seq] * HG;
    if (rows_total > a.short_rows || r >= rows_total) return;
    const int vd = a.vd;
    const size_t slot_stride = (size_t)a.n_seqs * a.nkv * 16 * 2;       // partials from one slot to the next
    float res[2][NDR];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp) {
        const size_t at0 = part_index(a, 0, seq, g, r, mp);
        float ms = -INFINITY, ls = 0.0f;
        if (lane < n_slots) {
            ms = a.part_ml[2 * (at0 + lane * slot_stride)];
            ls = a.part_ml[2 * (at0 + lane * slot_stride) + 1];
        }
        const float M = fb_warp_max(ls > 0.0f ? ms : -INFINITY);
        const float w = ls > 0.0f ? exp2f(ms - M) : 0.0f;               // this lane's slot's weight
        const float L = fb_warp_sum(w * ls);
#pragma unroll
        for (int d = 0; d < NDR; ++d) res[mp][d] = 0.0f;
        for (int s0 = 0; s0 < n_slots; s0 += 8) {
            float val[8][NDR];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float* po = a.part_o + (at0 + (size_t)min(s0 + u, n_slots - 1) * slot_stride) * vd;
#pragma unroll
                for (int d = 0; d < NDR; ++d) val[u][d] = lane + 32 * d < vd ? po[lane + 32 * d] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float wu = __shfl_sync(0xffffffffu, w, min(s0 + u, n_slots - 1));
                if (s0 + u < n_slots && wu > 0.0f) {
#pragma unroll
                    for (int d = 0; d < NDR; ++d) res[mp][d] = fmaf(wu, val[u][d], res[mp][d]);
                }
            }
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
        for (int d = 0; d < NDR; ++d) res[mp][d] *= inv;
    }
    float ss = 0.0f;
#pragma unroll
    for (int d = 0; d < NDR; ++d) {
        res[0][d] = lane + 32 * d < vd ? res[0][d] - a.lambda * res[1][d] : 0.0f;
        ss += res[0][d] * res[0][d];
    }
    ss = fb_warp_sum(ss);
    const int tok = a.seq_q_start[seq] + r / HG, h = g * HG + r % HG;
    const float f = a.out_scale * (a.gate ? a.gate[(size_t)tok * a.nh + h] : 1.0f) / sqrtf(ss / (float)vd + a.eps);
    __nv_bfloat16* op = a.out + (size_t)tok * a.out_stride + (size_t)h * vd;
#pragma unroll
    for (int d = 0; d < NDR; ++d)
        if (lane + 32 * d < vd) op[lane + 32 * d] = __float2bfloat16_rn(res[0][d] * f);
}

constexpr size_t SMEM_LIMIT = 200 * 1024;

size_t smem_bytes(int kd, int vd, bool split, int stages) {
    const int qrows = split ? 16 : 64;
    return ((size_t)2 * qrows * (kd + 8) + (size_t)stages * KT * (2 * kd + 8) + (size_t)stages * KT * (vd + 8)) *
           sizeof(__nv_bfloat16);
}
// Three tiles in shared memory where they fit (two in flight while one is used), else two.  The split arrangement
// streams the cache and keeps three only while two CTAs still fit on a multiprocessor.
int stages_for(int kd, int vd, bool split) {
    const size_t half = SMEM_LIMIT / 2 + 8 * 1024;                  // two CTAs of this size fit on a multiprocessor
    const size_t three = smem_bytes(kd, vd, split, 3);
    if (three <= half) return 3;
    if (smem_bytes(kd, vd, split, 2) <= half && vd <= 128) return 2;   // (larger values: one CTA by registers anyway)
    return three <= SMEM_LIMIT ? 3 : 2;
}

template <int KSTEPS, int VTILES, bool SPLIT, bool EXACT>
int launch_diff_mma(const DiffArgs& a, dim3 grid, cudaStream_t stream, int* resident) {
    const size_t smem = smem_bytes(a.kd, a.vd, SPLIT, a.n_stages);
    auto kern = diff_attention_mma_kernel<KSTEPS, VTILES, SPLIT, EXACT>;
    static bool raised[FB_MAX_DEVICES] = {};
    if (fb_needs_setup(raised)) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT) != cudaSuccess)
            return fb_fail(-1, "diff attention: cannot raise the shared-memory limit");
        fb_setup_done(raised);
    }
    if (smem > SMEM_LIMIT) return fb_fail(-1, "diff attention: %zu bytes of shared memory", smem);
    if (resident) {                       // asked only how many CTAs of this arrangement a multiprocessor holds
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 256, smem) != cudaSuccess || n < 1) n = 1;
        *resident = n;
        return 0;
    }
    fb_launch(kern, grid, 256, smem, stream, a);
    return fb_check_launch(SPLIT ? "diff_attention_split" : "diff_attention_portions");
}

template <bool SPLIT>
int dispatch_diff_mma(const DiffArgs& a, dim3 grid, cudaStream_t stream, int* resident = nullptr) {
#define FB_DIFF_MMA(KS, VT) return launch_diff_mma<KS, VT, SPLIT, false>(a, grid, stream, resident)
#define FB_DIFF_MMA_EXACT(KS, VT) \
    if (a.kd == KS * 16 && a.vd == VT * 8) return launch_diff_mma<KS, VT, SPLIT, true>(a, grid, stream, resident)
    FB_DIFF_MMA_EXACT(4, 16);           // key size 64 per map, value size 128
    FB_DIFF_MMA_EXACT(3, 12);           // 48 / 96
    FB_DIFF_MMA_EXACT(2, 8);            // 32 / 64
    FB_DIFF_MMA_EXACT(4, 8);            // 64 / 64
    FB_DIFF_MMA_EXACT(8, 16);           // 128 / 128
#undef FB_DIFF_MMA_EXACT
    if (a.kd <= 64) {
        if (a.vd <= 64) FB_DIFF_MMA(4, 8);
        if (a.vd <= 128) FB_DIFF_MMA(4, 16);
        FB_DIFF_MMA(4, 32);
    }
    if (a.vd <= 64) FB_DIFF_MMA(8, 8);
    if (a.vd <= 128) FB_DIFF_MMA(8, 16);
    FB_DIFF_MMA(8, 32);
#undef FB_DIFF_MMA
}

}  // namespace

// Scratch floats the split arrangement needs for `n_seqs` sequences with `n_splits` CTAs per (sequence, kv head).
FB_API long long fb_diff_attention_scratch_floats(int n_seqs, int nkv, int vd, int n_splits) {
    return (long long)n_splits * 4 * n_seqs * nkv * 16 * 2 * (vd + 2);
}

// How many CTAs per (sequence, key/value head) the split arrangement uses for a step of `n_seqs` sequences whose
// rows see at most `max_keys` keys: as many as are resident on the device at once (a CTA beyond that would run in a
// second round behind the others), at most one per key tile, at most 8 (four partials each: the combining kernel
// holds one partial's weight per lane).
FB_API int fb_diff_attention_splits(int n_seqs, int nkv, int max_keys, int kd, int vd) {
    if (kd % 16 || kd < 16 || kd > 128 || vd % 16 || vd < 16 || vd > 256) return 1;
    const int pairs = n_seqs * nkv > 0 ? n_seqs * nkv : 1;
    const int tiles = (max_keys + fb_attn::KT - 1) / fb_attn::KT + 1;
    DiffArgs a = {};
    a.kd = kd; a.vd = vd; a.n_stages = stages_for(kd, vd, true);
    int resident = 1;
    if (dispatch_diff_mma<true>(a, dim3(1), nullptr, &resident) != 0) resident = 1;
    int s = resident * fb_sm_count() / pairs;
    if (s > tiles) s = tiles;
    if (s > 8) s = 8;
    return s < 1 ? 1 : s;
}

FB_API int fb_diff_attention_mma(const void* q, long long q_stride, void* out, long long out_stride, const float* gate,
                                 const void* k_pool, const void* v_pool, int page_size, int n_pages,
                                 const int* block_table, int table_stride, const int* table_base,
                                 const int* seq_q_start, const int* seq_q_len, const int* seq_pos_start, int n_seqs,
                                 int max_q_len, int any_short, int any_long, int nh, int nkv, int kd, int vd,
                                 int window, float scale, float lambda, float eps, float out_scale, int n_splits,
                                 float* scratch, long long scratch_floats, int* status, cudaStream_t stream) {
    FB_REQUIRE(n_seqs >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0, "diff attention: bad head counts");
    FB_REQUIRE(kd % 16 == 0 && kd >= 16 && kd <= 128, "diff attention (mma): key size %d is not a multiple of 16 up to 128", kd);
    FB_REQUIRE(vd % 16 == 0 && vd >= 16 && vd <= 256, "diff attention (mma): value size %d is not a multiple of 16 up to 256", vd);
    FB_REQUIRE(page_size > 0 && n_pages > 0 && window >= 0 && eps > 0.0f, "diff attention: bad cache geometry or eps");
    FB_REQUIRE(scale > 0.0f, "diff attention (mma): the score scale must be positive");
    FB_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)out % 4 == 0 &&
               (uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0, "diff attention (mma): unaligned operands");
    FB_REQUIRE(n_seqs <= 65535 && nkv <= 65535, "diff attention: too many sequences or heads for one grid");
    if (n_seqs == 0) return 0;
    DiffArgs a;
    a.q = (const __nv_bfloat16*)q; a.q_stride = (long)q_stride;
    a.out = (__nv_bfloat16*)out; a.out_stride = (long)out_stride;
    a.gate = gate;
    a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
    a.page_size = page_size; a.n_pages = n_pages;
    a.page_shift = -1;
    for (int b = 0; b < 30; ++b) if ((1 << b) == page_size) a.page_shift = b;
    a.block_table = block_table; a.table_stride = table_stride; a.table_base = table_base;
    a.seq_q_start = seq_q_start; a.seq_q_len = seq_q_len; a.seq_pos_start = seq_pos_start;
    a.n_seqs = n_seqs; a.nh = nh; a.nkv = nkv; a.kd = kd; a.vd = vd; a.window = window;
    a.scale_log2e = scale * 1.4426950408889634f; a.lambda = lambda; a.eps = eps; a.out_scale = out_scale;
    a.short_rows = 16;
    a.n_splits = n_splits < 1 ? 1 : n_splits > 8 ? 8 : n_splits;
    a.part_o = nullptr; a.part_ml = nullptr;
    a.status = status;
    const int HG = nh / nkv;
    if (any_long) {
        a.n_stages = stages_for(kd, vd, false);
        const long rows = (long)max_q_len * HG;
        const int rc = dispatch_diff_mma<false>(a, dim3((unsigned)((rows + 63) / 64), nkv, n_seqs), stream);
        if (rc) return rc;
    }
    if (any_short) {
        const long long need = fb_diff_attention_scratch_floats(n_seqs, nkv, vd, a.n_splits);
        FB_REQUIRE(scratch && scratch_floats >= need, "diff attention: %lld floats of scratch wanted, %lld given", need,
                   scratch_floats);
        const size_t n_part = (size_t)a.n_splits * 4 * n_seqs * nkv * 16 * 2;
        a.part_o = scratch;
        a.part_ml = scratch + n_part * vd;
        a.n_stages = stages_for(kd, vd, true);
        const int rc = dispatch_diff_mma<true>(a, dim3(a.n_splits, nkv, n_seqs), stream);
        if (rc) return rc;
        const long items = (long)n_seqs * nkv * 16;
        const unsigned blocks = (unsigned)((items + 3) / 4);
        const int n_slots = a.n_splits * 4;
        if (vd <= 32) fb_launch((diff_attention_combine_kernel<1>), blocks, 128, 0, stream, a, n_slots);
        else if (vd <= 64) fb_launch((diff_attention_combine_kernel<2>), blocks, 128, 0, stream, a, n_slots);
        else if (vd <= 128) fb_launch((diff_attention_combine_kernel<4>), blocks, 128, 0, stream, a, n_slots);
        else fb_launch((diff_attention_combine_kernel<8>), blocks, 128, 0, stream, a, n_slots);
        return fb_check_launch("diff_attention_combine");
    }
    return 0;
}
