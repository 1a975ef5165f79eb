// layered_mixers.cuh -- more mechanisms of the layered runtime (layered.cu), beside those of layered_kernels.cuh and with the same
// rules: a kernel (or an epilogue) per mechanism, constants as arguments, fp32 for everything that is not a matrix-product operand,
// programmatic dependent launch at the top of every kernel, positions optionally read from a device word (captured decode step).
//
//   embedding            k_embed_pos (token row + learned position row)
//   norms                k_sandwich (residual update through a vector-gain RMS norm stored around zero, x += unit(d) (1 + w), and
//                        the next sublayer's input norm of the updated x, in one pass over the token)
//   rotary positions     k_rope ("rotate half" pairs over the first `dims` coordinates of each head, angles from a table built in
//                        double precision, optional scale on k after the rotation)
//   retention            k_retention_scan (linear attention with a fixed decay per head, no softmax, no denominator:
//                        S <- decay S + k v^T, o = S^T q; fp32 state [head][value column][key coordinate]; long portions as time
//                        segments side by side with k_retention_chain between the two passes; short portions rotate q and k while
//                        staging and finish the head's output in the last block), k_retention_out (per-head unit RMS of o times
//                        silu(gate))
//   window attention     k_qk_prepare (unit-RMS q and k per head, score scale and temperature folded into q, convolved k and its
//                        inverse RMS into the paged cache: the cached row is value AND, times that factor, key), k_window_attn
//                        (grouped-query softmax attention in a sliding window: soft cap, per-head distance slopes, scores mixed
//                        across heads before the softmax, sigmoid output gate)
//   selective scan       k_selective_scan (Mamba: S <- exp(dt A) S + dt x B, y = S C + D x, times silu(z); fp32 state [channel][n]),
//                        k_selective_scan_par (the same, parallel over time segments)
//   feed-forward         k_polynorm (a N(z) + b N(z^2) + c N(z^3) + e over the feed-forward width, N = unit RMS)
#pragma once
#include "layered_kernels.cuh"

namespace nb {
namespace lm {

__device__ __forceinline__ float siluf_(float z) { return z / (1.0f + expf(-z)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// x[t] = embed[tokens[t + off]] + ptab[pos0 + t + off],  off = *pos_ptr when given (a captured decode step), else 0
template <typename WT>
__global__ void k_embed_pos(const uint32_t *__restrict__ tokens, const uint32_t *__restrict__ pos_ptr, const WT *__restrict__ embed,
                            const WT *__restrict__ ptab, float *__restrict__ x, uint32_t E, uint32_t pos0) {
    pdl_enter();
    const uint32_t t = blockIdx.x, off = pos_ptr ? *pos_ptr : 0u;
    const WT *src = embed + (size_t)tokens[t + off] * E, *ps = ptab + (size_t)(pos0 + t + off) * E;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) x[(size_t)t * E + i] = wval(src + i) + wval(ps + i);
}

// One token per block.  With d: x[t] += d[t] / rms(d[t]) * (1 + w_post) (the sublayer's output norm and the residual sum); keep
// (optional) receives the updated x; with out: out[t] = x[t] / rms(x[t]) * (1 + w_pre), the input of the sublayer that follows.
// d2 (optional): a second branch of the sublayer, d + d2 is what gets normed.
struct SandwichArgs { float *x; const float *d; const float *w_post, *w_pre; float *out; float *keep; uint32_t T, E; float eps; const float *d2; };
__global__ void __launch_bounds__(1024) k_sandwich(const SandwichArgs a) {
    pdl_enter();
    __shared__ float red[32];
    const size_t row = (size_t)blockIdx.x * a.E;
    float *xt = a.x + row;
    if (a.d) {
        const float *dt = a.d + row, *d2 = a.d2 ? a.d2 + row : nullptr;
        float s = 0.0f;
        for (uint32_t i = threadIdx.x; i < a.E; i += blockDim.x) { const float v = d2 ? dt[i] + d2[i] : dt[i]; s = fmaf(v, v, s); }
        s = block_sum(s, red);
        const float rinv = 1.0f / sqrtf(s / (float)a.E + a.eps);
        for (uint32_t i = threadIdx.x; i < a.E; i += blockDim.x) {
            const float v = xt[i] + (d2 ? dt[i] + d2[i] : dt[i]) * rinv * (1.0f + a.w_post[i]);
            xt[i] = v;
            if (a.keep) a.keep[row + i] = v;
        }
    } else if (a.keep) {
        for (uint32_t i = threadIdx.x; i < a.E; i += blockDim.x) a.keep[row + i] = xt[i];
    }
    if (!a.out) return;
    float s = 0.0f;          // a thread reads back only what it wrote itself
    for (uint32_t i = threadIdx.x; i < a.E; i += blockDim.x) s = fmaf(xt[i], xt[i], s);
    s = block_sum(s, red);
    const float rinv = 1.0f / sqrtf(s / (float)a.E + a.eps);
    for (uint32_t i = threadIdx.x; i < a.E; i += blockDim.x) a.out[row + i] = xt[i] * rinv * (1.0f + a.w_pre[i]);
}

// Rotary positions in the "rotate half" layout on q and k of every head, in place: coordinate i < dims/2 pairs with i + dims/2,
// (u, v) -> (u cos - v sin, v cos + u sin) with the angle of tab[position][i] = (cos, sin); coordinates from `dims` on pass.  k is
// multiplied by kscale afterwards (1: none).  buf rows hold q at column q0 and k at column k0, H heads of D each.
struct RopeArgs { float *buf; uint32_t ld, q0, k0, T, H, D, dims, pos0; const float2 *tab; float kscale; const uint32_t *pos_ptr; };
__device__ __forceinline__ void rope_item(const RopeArgs &a, float *q, float *k, uint32_t pos, uint32_t i) {
    const uint32_t half = a.tab ? a.dims / 2u : 0u;
    if (i < half) {
        const float2 cs = a.tab[(size_t)pos * half + i];
        const float qu = q[i], qv = q[i + half], ku = k[i], kv = k[i + half];
        q[i] = qu * cs.x - qv * cs.y; q[i + half] = qv * cs.x + qu * cs.y;
        k[i] = (ku * cs.x - kv * cs.y) * a.kscale; k[i + half] = (kv * cs.x + ku * cs.y) * a.kscale;
    } else {
        k[i + half] *= a.kscale;
    }
}
__global__ void k_rope(const RopeArgs a) {
    pdl_enter();
    const uint32_t per = a.D - (a.tab ? a.dims / 2u : 0u), pos = a.pos0 + (a.pos_ptr ? *a.pos_ptr : 0u);
    const size_t total = (size_t)a.T * a.H * per;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(idx / ((size_t)a.H * per)), rem = (uint32_t)(idx % ((size_t)a.H * per)), h = rem / per, i = rem % per;
        float *row = a.buf + (size_t)t * a.ld;
        rope_item(a, row + a.q0 + h * a.D, row + a.k0 + h * a.D, pos + t, i);
    }
}

// Retention, token by token.  A block of 8 warps owns 8 x CPW value columns of head h = blockIdx.y (a warp CPW of them) and
// keeps S[h][:, j] in registers (lane l holds key coordinates l, l + 32, ...); per token S <- decay_h S + k v_j and o_j = S . q.
// q, k and v of 32 (or 16) tokens at a time are staged in shared memory, read there by every warp.
// p rows hold q at q0, k at k0, v at v0.  The state is [H][VD][D] fp32; o is [T][H * VD].
// Rotary positions are applied while q and k are staged (rot_tab given: the table of k_rope; k times kscale afterwards in any case).
// finish (short portions): the block that draws the last ticket of its head (one zeroed counter per head) also does k_retention_out's
// work for the head: out = o / rms(o) * silu(g).
struct RetentionArgs { const float *p; uint32_t ld, q0, k0, v0; const float *decay; float *S; float *o; uint32_t T, H, D, VD;
                       uint32_t dims, pos0; const float2 *rot_tab; float kscale; const uint32_t *pos_ptr;
                       uint32_t finish; const float *g; uint32_t ldg; float *out; float eps; uint32_t *tickets;
                       // Long portions run parallel over time: gridDim.z segments of seg_len tokens.  mode 1: every segment starts from zero
                       // and leaves the state it builds in seg_S[segment] (no outputs); k_retention_chain turns those into the states each
                       // segment starts from (and the slot's state after the portion); mode 2: every segment starts from seg_S[segment]
                       // and writes its outputs (the slot's state is not touched).  mode 0: one pass over all tokens from and to S.
                       uint32_t mode, seg_len; float *seg_S; };
// CPW: value columns per warp (4: fewest shared-memory reads per FMA; 1: most warps, for models whose heads x columns would leave SMs idle)
template <int DCH, int CPW>
__global__ void __launch_bounds__(256) k_retention_scan(const RetentionArgs a) {
    pdl_enter();
    constexpr uint32_t kRetCpw = CPW, kRetCols = 8 * CPW, kRetTile = DCH <= 4 ? 32 : 16;          // tokens staged at a time
    __shared__ float qs[kRetTile][DCH * 32], ks[kRetTile][DCH * 32], vs[kRetTile][kRetCols];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, h = blockIdx.y, j0 = blockIdx.x * kRetCols, jw = j0 + warp * kRetCpw;
    float *Sio = a.mode ? a.seg_S + (size_t)blockIdx.z * a.H * a.VD * a.D : a.S;          // where this block's state comes from and goes to
    const uint32_t t_lo = a.mode ? blockIdx.z * a.seg_len : 0u, t_hi = a.mode ? min(a.T, t_lo + a.seg_len) : a.T;
    float S[kRetCpw][DCH];
#pragma unroll
    for (uint32_t i = 0; i < kRetCpw; i++)
#pragma unroll
        for (int c = 0; c < DCH; c++) { const uint32_t d = lane + 32u * c; S[i][c] = (a.mode != 1u && jw + i < a.VD && d < a.D) ? Sio[((size_t)h * a.VD + jw + i) * a.D + d] : 0.0f; }
    const float g = a.decay[h];
    const uint32_t half = a.rot_tab ? a.dims / 2u : 0u, pos = a.pos0 + (a.pos_ptr ? *a.pos_ptr : 0u);
    for (uint32_t t0 = t_lo; t0 < t_hi; t0 += kRetTile) {
        const uint32_t nt = min(kRetTile, t_hi - t0);
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < nt * DCH * 32u; i += blockDim.x) {
            const uint32_t t = i / (DCH * 32u), d = i % (DCH * 32u);
            const float *qr = a.p + (size_t)(t0 + t) * a.ld + a.q0 + h * a.D, *kr = a.p + (size_t)(t0 + t) * a.ld + a.k0 + h * a.D;
            float qv = 0.0f, kv = 0.0f;
            if (d < a.D) {
                qv = a.mode == 1u ? 0.0f : qr[d]; kv = kr[d];          // the state-only pass needs no q
                if (d < 2u * half) {          // the pair (i, i + half): (u, v) -> (u cos - v sin, v cos + u sin)
                    const bool lo = d < half;
                    const float2 cs = a.rot_tab[(size_t)(pos + t0 + t) * half + (lo ? d : d - half)];
                    const float qo = lo ? -qr[d + half] : qr[d - half], ko = lo ? -kr[d + half] : kr[d - half];
                    qv = qv * cs.x + qo * cs.y; kv = kv * cs.x + ko * cs.y;
                }
                kv *= a.kscale;
            }
            qs[t][d] = qv; ks[t][d] = kv;
        }
        for (uint32_t i = threadIdx.x; i < nt * kRetCols; i += blockDim.x) {
            const uint32_t t = i / kRetCols, j = i % kRetCols;
            vs[t][j] = j0 + j < a.VD ? a.p[(size_t)(t0 + t) * a.ld + a.v0 + h * a.VD + j0 + j] : 0.0f;
        }
        __syncthreads();
        if (a.mode == 1u) {          // the first pass of a long portion only builds states
            for (uint32_t t = 0; t < nt; t++) {
                float v[kRetCpw];
#pragma unroll
                for (uint32_t i = 0; i < kRetCpw; i++) v[i] = vs[t][warp * kRetCpw + i];
#pragma unroll
                for (int c = 0; c < DCH; c++) {
                    const float kd = ks[t][lane + 32 * c];
#pragma unroll
                    for (uint32_t i = 0; i < kRetCpw; i++) S[i][c] = fmaf(g, S[i][c], kd * v[i]);
                }
            }
            continue;
        }
        for (uint32_t t = 0; t < nt; t++) {
            float acc[kRetCpw], v[kRetCpw];
#pragma unroll
            for (uint32_t i = 0; i < kRetCpw; i++) { acc[i] = 0.0f; v[i] = vs[t][warp * kRetCpw + i]; }
#pragma unroll
            for (int c = 0; c < DCH; c++) {
                const float kd = ks[t][lane + 32 * c], qd = qs[t][lane + 32 * c];
#pragma unroll
                for (uint32_t i = 0; i < kRetCpw; i++) { S[i][c] = fmaf(g, S[i][c], kd * v[i]); acc[i] = fmaf(S[i][c], qd, acc[i]); }
            }
            float *orow = a.o + (size_t)(t0 + t) * a.H * a.VD + h * a.VD + jw;
            if (kRetCpw == 4) {
                // four sums over the warp with six shuffles: halves of the warp trade two columns, quarters one, then eight lanes add up;
                // lanes 0, 8, 16, 24 end with columns 0, 1, 2, 3
                const bool h16 = lane & 16u, h8 = lane & 8u;
                float k0 = (h16 ? acc[2] : acc[0]) + __shfl_xor_sync(0xffffffffu, h16 ? acc[0] : acc[2], 16);
                float k1 = (h16 ? acc[3] : acc[1]) + __shfl_xor_sync(0xffffffffu, h16 ? acc[1] : acc[3], 16);
                float k = (h8 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, h8 ? k0 : k1, 8);
                k += __shfl_xor_sync(0xffffffffu, k, 4); k += __shfl_xor_sync(0xffffffffu, k, 2); k += __shfl_xor_sync(0xffffffffu, k, 1);
                const uint32_t col = lane >> 3;
                if ((lane & 7u) == 0 && jw + col < a.VD) orow[col] = k;
            } else {
#pragma unroll
                for (uint32_t i = 0; i < kRetCpw; i++) acc[i] = warp_sum(acc[i]);
                float mine = acc[0];
#pragma unroll
                for (uint32_t i = 1; i < kRetCpw; i++) if (lane == i) mine = acc[i];
                if (lane < kRetCpw && jw + lane < a.VD) orow[lane] = mine;
            }
        }
    }
    if (a.mode == 2u) return;
#pragma unroll
    for (uint32_t i = 0; i < kRetCpw; i++)
#pragma unroll
        for (int c = 0; c < DCH; c++) { const uint32_t d = lane + 32u * c; if (jw + i < a.VD && d < a.D) Sio[((size_t)h * a.VD + jw + i) * a.D + d] = S[i][c]; }
    if (!a.finish) return;
    __shared__ uint32_t last_s;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t got = atomicAdd(a.tickets + h, 1u);
        last_s = got + 1u == gridDim.x;
        if (last_s) a.tickets[h] = 0u;              // ready for the next launch
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    for (uint32_t t = warp; t < a.T; t += blockDim.x >> 5) {          // a warp per token: the head's o over all value columns
        const float *o = a.o + ((size_t)t * a.H + h) * a.VD, *gp = a.g + (size_t)t * a.ldg + h * a.VD;
        float s = 0.0f;
        for (uint32_t i = lane; i < a.VD; i += 32u) { const float v = __ldcg(o + i); s = fmaf(v, v, s); }
        s = warp_sum(s);
        const float rinv = 1.0f / sqrtf(s / (float)a.VD + a.eps);
        float *out = a.out + ((size_t)t * a.H + h) * a.VD;
        for (uint32_t i = lane; i < a.VD; i += 32u) out[i] = __ldcg(o + i) * rinv * siluf_(gp[i]);
    }
}

// Between the two passes of a long portion: seg_S[s] holds what segment s built from zero; it becomes the state segment s starts
// from, S_s = decay^len(s-1) S_(s-1) + built(s-1), S_0 = the slot's state, which in turn becomes the state after the last segment.
struct RetChainArgs { float *S; float *seg_S; const float *decay; uint32_t H, D, VD, T, seg_len, nseg; };      // nseg <= 8
__global__ void __launch_bounds__(256) k_retention_chain(const RetChainArgs a) {
    pdl_enter();
    const uint32_t per = a.VD * a.D, h = blockIdx.y;          // grid = (blocks over a head's state, heads)
    const size_t total = (size_t)per * a.H;
    const float g = a.decay[h], lg = log2f(g);
    for (uint32_t j = blockIdx.x * blockDim.x + threadIdx.x; j < per; j += gridDim.x * blockDim.x) {
        const size_t i = (size_t)h * per + j;
        float built[8];
#pragma unroll
        for (uint32_t sg = 0; sg < 8; sg++) built[sg] = sg < a.nseg ? a.seg_S[(size_t)sg * total + i] : 0.0f;
        float s = a.S[i];
#pragma unroll
        for (uint32_t sg = 0; sg < 8; sg++) {
            if (sg >= a.nseg) break;
            const uint32_t len = min(a.T, (sg + 1u) * a.seg_len) - sg * a.seg_len;
            a.seg_S[(size_t)sg * total + i] = s;
            s = fmaf(exp2f((float)len * lg), s, built[sg]);          // decay^len
        }
        a.S[i] = s;
    }
}

// each head's o divided by its root mean square over the value columns, times silu(gate): a warp per (token, head)
struct RetOutArgs { const float *o; const float *g; uint32_t ldg; float *out; uint32_t T, H, VD; float eps; };
__global__ void __launch_bounds__(256) k_retention_out(const RetOutArgs a) {
    pdl_enter();
    const uint32_t warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (warp >= a.T * a.H) return;
    const uint32_t t = warp / a.H, h = warp % a.H;
    const float *o = a.o + ((size_t)t * a.H + h) * a.VD, *g = a.g + (size_t)t * a.ldg + h * a.VD;
    float s = 0.0f;
    for (uint32_t i = lane; i < a.VD; i += 32u) s = fmaf(o[i], o[i], s);
    s = warp_sum(s);
    const float rinv = 1.0f / sqrtf(s / (float)a.VD + a.eps);
    float *out = a.out + ((size_t)t * a.H + h) * a.VD;
    for (uint32_t i = lane; i < a.VD; i += 32u) out[i] = o[i] * rinv * siluf_(g[i]);
}

// Window attention, first step.  One block per token, a warp per head: q (H heads) becomes unit-RMS times qmul[h] (the score scale
// and the head's temperature), in place; k (G heads) goes into the token's cache row as it is -- it is the value -- followed by the
// G factors 1 / rms(k_g), so that the key is the row times its factor.  Row length RL = G * D + G rounded up to 4 floats.
struct QkPrepArgs { float *q; uint32_t ldq; const float *k; uint32_t ldk; const float *temp; float scale; float *cache; const uint32_t *table;
                    uint32_t H, G, D, RL, pos0; float eps; const uint32_t *pos_ptr; };
__global__ void __launch_bounds__(256) k_qk_prepare(const QkPrepArgs a) {
    pdl_enter();
    const uint32_t t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, nw = blockDim.x >> 5;
    const uint32_t pos = a.pos0 + t + (a.pos_ptr ? *a.pos_ptr : 0u);
    float *row = a.cache + ((size_t)a.table[pos / kPage] * kPage + pos % kPage) * a.RL;
    for (uint32_t job = warp; job < a.H + a.G; job += nw) {
        if (job < a.H) {
            float *q = a.q + (size_t)t * a.ldq + job * a.D;
            float s = 0.0f;
            for (uint32_t i = lane; i < a.D; i += 32u) s = fmaf(q[i], q[i], s);
            s = warp_sum(s);
            const float f = 1.0f / sqrtf(s / (float)a.D + a.eps) * (a.scale * a.temp[job]);
            for (uint32_t i = lane; i < a.D; i += 32u) q[i] *= f;
        } else {
            const uint32_t g = job - a.H;
            const float *k = a.k + (size_t)t * a.ldk + g * a.D;
            float s = 0.0f;
            for (uint32_t i = lane; i < a.D; i += 32u) { const float v = k[i]; s = fmaf(v, v, s); row[g * a.D + i] = v; }
            s = warp_sum(s);
            if (lane == 0) row[a.G * a.D + g] = 1.0f / sqrtf(s / (float)a.D + a.eps);
        }
    }
    if (threadIdx.x < a.RL - (a.G * a.D + a.G)) row[a.G * a.D + a.G + threadIdx.x] = 0.0f;      // the padding of the row
}

// Sliding-window softmax attention with grouped keys/values whose scores are mixed across heads.  For query position i and key
// position j, 0 <= i - j < window:
//     s_h = q'_h . k_j,g(h)                      q' already carries scale x temperature; k = cached row x its 1/rms factor
//     s_h <- cap tanh(s_h / cap)                 (cap 0: none)
//     s_h <- s_h - slope_h (i - j)
//     s_h <- sum_g talk[h][g] s_g                (talk null: none)       -- needs every head of the (i, j) pair in one block
//     p_h = softmax_j s_h,   o_h = sum_j p_h v_j,g(h),   out = o_h x sigmoid(gate_h)   (gate null: none)
// grid = query tiles of QT tokens; blockDim = 32 x ceil(H / HS): a warp owns HS heads (h = warp + hs x warps).  A key tile is one
// cache page: phase 1 writes every head's capped, sloped score of the tile's 32 keys to shared memory (lanes = keys), phase 2 mixes
// them, runs the online softmax and accumulates the values (lanes = value columns).  Everything in fp32.
struct WinAttnArgs {
    const float *q; uint32_t ldq; const float *cache; const uint32_t *table; const float *gate; uint32_t ldg;
    const float *talk, *slopes; float *out;
    uint32_t T, H, G, D, RL, pos0, window; float softcap; const uint32_t *pos_ptr;
    // key splits (short portions): gridDim.y = nsplit blocks share a query tile's key pages and write partial (o, m, l) triples to
    // part [T][nsplit][H][D + 2]; the block that draws the last ticket of its query tile (one zeroed counter each) merges them
    uint32_t nsplit; float *part; uint32_t *tickets;
};
__host__ __device__ inline uint32_t win_attn_ldc(uint32_t RL) { return ((RL / 4u) & 1u) ? RL : RL + 4u; }      // rows of an odd number of 16-byte units
__host__ __device__ inline uint32_t win_attn_qs(uint32_t H, uint32_t D, uint32_t qt) { return (qt * H * D + 3u) & ~3u; }
inline size_t win_attn_smem(uint32_t H, uint32_t D, uint32_t RL, uint32_t qt) {
    return ((size_t)win_attn_qs(H, D, qt) + (size_t)kPage * win_attn_ldc(RL) + (size_t)qt * H * 32u + (size_t)H * H + H) * 4;
}
template <int VCH, int QT, int HS>
__global__ void __launch_bounds__(512) k_window_attn(const WinAttnArgs a) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const uint32_t nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t H = a.H, D = a.D, HD = H * D, rep = H / a.G, GD = a.G * D;
    const uint32_t tq0 = blockIdx.x * QT, nq = min((uint32_t)QT, a.T - tq0);
    const uint32_t LDC = win_attn_ldc(a.RL);
    float *q_s = sm;                                       // [QT][H * D]
    float *c_s = q_s + win_attn_qs(H, D, QT);              // [kPage][LDC]
    float *s_s = c_s + kPage * LDC;                        // [QT][H][32]
    float *t_s = s_s + QT * H * 32u;                       // [H][H], then the H slopes
    const bool vec = (D % 4u) == 0;
    for (uint32_t i = threadIdx.x; i < H * H; i += blockDim.x) t_s[i] = a.talk ? a.talk[i] : 0.0f;
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) t_s[H * H + i] = a.slopes ? a.slopes[i] : 0.0f;
    for (uint32_t i = threadIdx.x; i < QT * HD; i += blockDim.x) {
        const uint32_t qi = i / HD;
        q_s[i] = qi < nq ? a.q[(size_t)(tq0 + qi) * a.ldq + i % HD] : 0.0f;
    }
    const uint32_t p0 = a.pos0 + (a.pos_ptr ? *a.pos_ptr : 0u) + tq0, last = p0 + nq - 1u;      // positions of the tile's first and last query
    const uint32_t tile_lo = p0 + 1u > a.window ? (p0 + 1u - a.window) / kPage : 0u, tile_hi = last / kPage;
    const uint32_t tps = (tile_hi - tile_lo + a.nsplit) / a.nsplit;                         // key pages per split
    const uint32_t my_lo = tile_lo + blockIdx.y * tps, my_hi = min(tile_hi + 1u, my_lo + tps);
    float m[HS][QT], l[HS][QT], o[HS][QT][VCH];
#pragma unroll
    for (int hs = 0; hs < HS; hs++)
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            m[hs][qi] = -INFINITY; l[hs][qi] = 0.0f;
#pragma unroll
            for (int c = 0; c < VCH; c++) o[hs][qi][c] = 0.0f;
        }
    for (uint32_t tile = my_lo; tile < my_hi; tile++) {
        __syncthreads();
        const uint32_t nk = min(kPage, last + 1u - tile * kPage);      // keys of this page that exist so far
        {
            const float4 *src4 = reinterpret_cast<const float4 *>(a.cache + (size_t)a.table[tile] * kPage * a.RL);
            const uint32_t rl4 = a.RL / 4u, n4 = nk * rl4;
            for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x)
                *reinterpret_cast<float4 *>(c_s + (i / rl4) * LDC + (i % rl4) * 4u) = __ldg(src4 + i);
        }
        __syncthreads();
        const uint32_t jg = tile * kPage + lane;           // this lane's key position
        uint32_t seen = 0;                                 // bit qi: query qi sees this lane's key
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            const uint32_t pi = p0 + qi;
            if ((uint32_t)qi < nq && jg <= pi && pi - jg < a.window) seen |= 1u << qi;
        }
        // phase 1: capped, sloped scores of every head
#pragma unroll
        for (int hs = 0; hs < HS; hs++) {
            const uint32_t h = warp + hs * nw;
            if (h >= H) continue;
            const uint32_t kv = h / rep;
            const float *cr = c_s + lane * LDC + kv * D;
            float sc[QT];
#pragma unroll
            for (int qi = 0; qi < QT; qi++) sc[qi] = 0.0f;
            if (vec) {
                const float4 *c4 = reinterpret_cast<const float4 *>(cr);
                for (uint32_t r4 = 0; r4 < D / 4u; r4++) {
                    const float4 cv = c4[r4];
#pragma unroll
                    for (int qi = 0; qi < QT; qi++) {
                        const float4 qv = reinterpret_cast<const float4 *>(q_s + (size_t)qi * HD + h * D)[r4];
                        sc[qi] = fmaf(qv.w, cv.w, fmaf(qv.z, cv.z, fmaf(qv.y, cv.y, fmaf(qv.x, cv.x, sc[qi]))));
                    }
                }
            } else {
                for (uint32_t r = 0; r < D; r++) {
                    const float cv = cr[r];
#pragma unroll
                    for (int qi = 0; qi < QT; qi++) sc[qi] = fmaf(q_s[(size_t)qi * HD + h * D + r], cv, sc[qi]);
                }
            }
            const float rinv = c_s[lane * LDC + GD + kv], slope = t_s[H * H + h];
#pragma unroll
            for (int qi = 0; qi < QT; qi++) {
                float s = sc[qi] * rinv;
                if (a.softcap > 0.0f) s = a.softcap * tanhf(s / a.softcap);
                s -= slope * (float)(int32_t)(p0 + qi - jg);
                s_s[((size_t)qi * H + h) * 32u + lane] = ((seen >> qi) & 1u) ? s : 0.0f;      // rows past nk hold stale numbers: select, never multiply
            }
        }
        __syncthreads();
        // phase 2: mix across heads, online softmax, values
        const uint32_t j_lo = p0 + 1u > a.window + tile * kPage ? p0 + 1u - a.window - tile * kPage : 0u;      // keys before the first query's window
#pragma unroll
        for (int hs = 0; hs < HS; hs++) {
            const uint32_t h = warp + hs * nw;
            if (h >= H) continue;
            const uint32_t kv = h / rep;
            float p[QT];
#pragma unroll
            for (int qi = 0; qi < QT; qi++) {
                float s;
                if (a.talk) {
                    s = 0.0f;
                    for (uint32_t g = 0; g < H; g++) s = fmaf(t_s[h * H + g], s_s[((size_t)qi * H + g) * 32u + lane], s);
                } else s = s_s[((size_t)qi * H + h) * 32u + lane];
                const bool sn = (seen >> qi) & 1u;
                s = sn ? s : -INFINITY;
                float tm = s;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, off));
                const float mn = fmaxf(m[hs][qi], tm);
                const float corr = mn == -INFINITY ? 1.0f : expf(m[hs][qi] - mn);
                p[qi] = sn ? expf(s - mn) : 0.0f;
                const float ps = warp_sum(p[qi]);
                l[hs][qi] = l[hs][qi] * corr + ps;
                m[hs][qi] = mn;
#pragma unroll
                for (int c = 0; c < VCH; c++) o[hs][qi][c] *= corr;
            }
            for (uint32_t j = j_lo; j < nk; j++) {
                float pj[QT];
#pragma unroll
                for (int qi = 0; qi < QT; qi++) pj[qi] = __shfl_sync(0xffffffffu, p[qi], j);
                const float *cj = c_s + j * LDC + kv * D;
#pragma unroll
                for (int c = 0; c < VCH; c++) {
                    const uint32_t r = lane + 32u * c;
                    if (r < D) {
                        const float cv = cj[r];
#pragma unroll
                        for (int qi = 0; qi < QT; qi++) o[hs][qi][c] = fmaf(pj[qi], cv, o[hs][qi][c]);
                    }
                }
            }
        }
    }
    if (a.nsplit == 1) {
#pragma unroll
        for (int hs = 0; hs < HS; hs++) {
            const uint32_t h = warp + hs * nw;
            if (h >= H) continue;
#pragma unroll
            for (int qi = 0; qi < QT; qi++) {
                if ((uint32_t)qi >= nq) continue;
                const size_t t = tq0 + qi;
                const float inv = 1.0f / l[hs][qi];
#pragma unroll
                for (int c = 0; c < VCH; c++) {
                    const uint32_t r = lane + 32u * c;
                    if (r >= D) continue;
                    float v = o[hs][qi][c] * inv;
                    if (a.gate) v *= sigmoidf_(a.gate[t * a.ldg + h * D + r]);
                    a.out[t * HD + h * D + r] = v;
                }
            }
        }
        return;
    }
    // key splits: partial triples, then the last block of the query tile merges
    //   out = sum_s e^{m_s - M} o_s / sum_s e^{m_s - M} l_s   over the splits that saw keys
#pragma unroll
    for (int hs = 0; hs < HS; hs++) {
        const uint32_t h = warp + hs * nw;
        if (h >= H) continue;
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            if ((uint32_t)qi >= nq) continue;
            float *dst = a.part + (((size_t)(tq0 + qi) * a.nsplit + blockIdx.y) * H + h) * (D + 2u);
#pragma unroll
            for (int c = 0; c < VCH; c++) { const uint32_t r = lane + 32u * c; if (r < D) dst[r] = o[hs][qi][c]; }
            if (lane == 0) { dst[D] = m[hs][qi]; dst[D + 1u] = l[hs][qi]; }
        }
    }
    __shared__ uint32_t last_s;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t *tk = a.tickets + blockIdx.x;
        const uint32_t got = atomicAdd(tk, 1u);
        last_s = got + 1u == a.nsplit;
        if (last_s) *tk = 0u;              // ready for the next launch
    }
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    const size_t stride = (size_t)H * (D + 2u);
#pragma unroll
    for (int hs = 0; hs < HS; hs++) {
        const uint32_t h = warp + hs * nw;
        if (h >= H) continue;
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            if ((uint32_t)qi >= nq) continue;
            const size_t t = tq0 + qi;
            const float *base = a.part + ((size_t)t * a.nsplit * H + h) * (D + 2u);
            const bool live = lane < a.nsplit;
            const float ls = live ? __ldcg(base + lane * stride + D + 1u) : 0.0f;
            const float ms = (live && ls > 0.0f) ? __ldcg(base + lane * stride + D) : -INFINITY;
            float M = ms;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
            const float w = ls > 0.0f ? expf(ms - M) : 0.0f;
            const float Lsum = warp_sum(w * ls);
            float acc[VCH];
#pragma unroll
            for (int c = 0; c < VCH; c++) acc[c] = 0.0f;
            for (uint32_t sp = 0; sp < a.nsplit; sp++) {
                const float ws = __shfl_sync(0xffffffffu, w, sp);
                if (ws == 0.0f) continue;          // a split without keys wrote nothing of weight (uniform over the warp)
#pragma unroll
                for (int c = 0; c < VCH; c++) { const uint32_t r = lane + 32u * c; if (r < D) acc[c] = fmaf(ws, __ldcg(base + sp * stride + r), acc[c]); }
            }
            const float inv = 1.0f / Lsum;
#pragma unroll
            for (int c = 0; c < VCH; c++) {
                const uint32_t r = lane + 32u * c;
                if (r >= D) continue;
                float v = acc[c] * inv;
                if (a.gate) v *= sigmoidf_(a.gate[t * a.ldg + h * D + r]);
                a.out[t * HD + h * D + r] = v;
            }
        }
    }
}

// Selective scan (Mamba), token by token.  A group of LG lanes owns channel c; lane g of the group holds the states n = 4g .. 4g + 3
// (their B and C are one 16-byte load each where the row layout allows).  Per token:  S[c][n] <- exp(dt_c A[c][n]) S[c][n] + (dt_c x_c) B_n,  y_c = sum_n S[c][n] C_n + D_c x_c,
// out = y_c silu(z_c).  dt [T][C] is the step size after its softplus, x [T][C] the convolved, activated input, B and C sit in the
// rows of bc at columns b0 and c0, A = -exp(A_log) [C][N].
// exp(z) S + b for z <= 0.  A slowly decaying state takes thousands of these steps, and the error of expf (two units in the last
// place of a number near 1) would be several times the rounding of the sum itself; for small |z| the decay is taken as 1 + expm1(z),
// whose error is relative to |z|, and applied as S + (expm1(z) S + b).
__device__ __forceinline__ float decay_drive(float z, float S, float b) {
    if (z > -0.25f) {          // expm1(z) by its series to z^7 / 7!: the first term left out is below 2e-9 |z| here
        const float p = fmaf(z, fmaf(z, fmaf(z, fmaf(z, fmaf(z, fmaf(z, 1.0f / 5040.0f, 1.0f / 720.0f), 1.0f / 120.0f), 1.0f / 24.0f), 1.0f / 6.0f), 0.5f), 1.0f);
        return S + fmaf(z * p, S, b);
    }
    return fmaf(expf(z), S, b);
}
// With dt_w (fp32 [C][R], short portions) the step size is made here: dt_c = softplus(dt_w[c] . bc[t][0..R) + dt_b[c]); round_a rounds
// that operand to bf16 first, as a tensor-core product of the same numbers would.
// four consecutive values row[n0 .. n0 + 4) of a [.., N] row (zeros past N): one 16-byte load where the layout allows it
__device__ __forceinline__ void load4(const float *__restrict__ p, uint32_t n0, uint32_t N, bool vec, float (&v)[4]) {
    if (vec && n0 + 4u <= N) { const float4 q = *reinterpret_cast<const float4 *>(p + n0); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
    else {
#pragma unroll
        for (uint32_t k = 0; k < 4; k++) v[k] = n0 + k < N ? p[n0 + k] : 0.0f;
    }
}
struct SelScanArgs { const float *dt; const float *x; const float *bc; uint32_t ldb, b0, c0; const float *A, *Dv; const float *z; uint32_t ldz;
                     float *S; float *y; uint32_t T, C, N; const float *dt_w, *dt_b; uint32_t R, round_a; };
template <int LG>
__global__ void __launch_bounds__(256) k_selective_scan(const SelScanArgs a) {
    pdl_enter();
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x, c = gid / LG, g = gid % LG;
    const bool live = c < a.C;          // dead lanes keep running: the group sums are warp shuffles
    const bool vec4 = ((a.b0 | a.c0 | a.ldb) & 3u) == 0 && (reinterpret_cast<uintptr_t>(a.bc) & 15u) == 0;
    float S[4], Av[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t n = g * 4u + k;
        const bool ok = live && n < a.N;
        S[k] = ok ? a.S[(size_t)c * a.N + n] : 0.0f;
        Av[k] = ok ? a.A[(size_t)c * a.N + n] : 0.0f;
    }
    const float Dc = live ? a.Dv[c] : 0.0f;
    for (uint32_t t = 0; t < a.T; t++) {
        const float *row = a.bc + (size_t)t * a.ldb;
        float dtc;
        if (a.dt_w) {          // the group's lanes share the dot product of length R
            float s = 0.0f;
            if (live) for (uint32_t r = g; r < a.R; r += LG) { const float v = row[r]; s = fmaf(a.dt_w[(size_t)c * a.R + r], a.round_a ? round_bf16(v) : v, s); }
#pragma unroll
            for (int off = LG / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            dtc = live ? softplusf_(s + a.dt_b[c]) : 0.0f;
        } else dtc = live ? a.dt[(size_t)t * a.C + c] : 0.0f;
        const float xv = live ? a.x[(size_t)t * a.C + c] : 0.0f, dx = dtc * xv;
        float acc = 0.0f, Bv[4], Cv[4];
        load4(row + a.b0, g * 4u, a.N, vec4, Bv); load4(row + a.c0, g * 4u, a.N, vec4, Cv);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            if (g * 4u + k < a.N) {
                S[k] = decay_drive(dtc * Av[k], S[k], dx * Bv[k]);
                acc = fmaf(S[k], Cv[k], acc);
            }
        }
#pragma unroll
        for (int off = LG / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (live && g == 0) a.y[(size_t)t * a.C + c] = (acc + Dc * xv) * siluf_(a.z[(size_t)t * a.ldz + c]);
    }
    if (live)
#pragma unroll
        for (int k = 0; k < 4; k++) { const uint32_t n = g * 4u + k; if (n < a.N) a.S[(size_t)c * a.N + n] = S[k]; }
}

// The same scan for long portions, parallel over time: blockDim = (32, segments).  A thread first composes its time segment's
// affine map S -> P S + Q per state (P = exp of the summed exponents), the segment-0 threads chain the maps to every segment's entry
// state (and the portion's final state), then each thread replays its segment from its entry state and writes the outputs.
// STAGE: the block first brings dt, x and z of its 32 / LG channels for the whole portion into (dynamic) shared memory, all loads in
// flight at once, and both passes read them there; sel_scan_stage_bytes says how much that takes.  (Staging the B rows in place of z,
// which is read only once, measured slower: 308 us against 275 us on a 1024-token chunk of 4096 channels.)
inline size_t sel_scan_stage_bytes(uint32_t T, uint32_t LG) { return (size_t)3 * T * (32u / LG) * 4; }
template <int LG, bool STAGE>
__global__ void __launch_bounds__(1024) k_selective_scan_par(const SelScanArgs a) {
    pdl_enter();
    __shared__ float P[32][32][4], Q[32][32][4];
    extern __shared__ __align__(16) float stage[];
    constexpr uint32_t CH = 32u / LG;
    float *dts = stage, *xs = stage + (size_t)a.T * CH, *zst = stage + (size_t)2 * a.T * CH;
    if (STAGE) {
        const uint32_t tid = threadIdx.y * 32u + threadIdx.x, nthr = blockDim.y * 32u, c0 = blockIdx.x * CH;
        for (uint32_t i = tid; i < a.T * CH; i += nthr) {
            const uint32_t t = i / CH, cc = c0 + i % CH;
            const bool ok = cc < a.C;
            dts[i] = ok ? a.dt[(size_t)t * a.C + cc] : 0.0f;
            xs[i] = ok ? a.x[(size_t)t * a.C + cc] : 0.0f;
            zst[i] = ok ? a.z[(size_t)t * a.ldz + cc] : 0.0f;
        }
        __syncthreads();
    }
    const uint32_t x = threadIdx.x, seg = threadIdx.y, nseg = blockDim.y, gid = blockIdx.x * 32u + x, c = gid / LG, g = gid % LG;
    const uint32_t Ls = (a.T + nseg - 1u) / nseg, t0 = min(a.T, seg * Ls), t1 = min(a.T, t0 + Ls);
    // inputs and output never overlap: with that said, the loads of the unrolled steps can all be issued before the first store
    const float *__restrict__ dtp = a.dt, *__restrict__ xp = a.x, *__restrict__ bcp = a.bc, *__restrict__ zp = a.z;
    float *__restrict__ yp = a.y;
    const bool live = c < a.C;
    const bool vec4 = ((a.b0 | a.c0 | a.ldb) & 3u) == 0 && (reinterpret_cast<uintptr_t>(a.bc) & 15u) == 0;
    float Av[4];
#pragma unroll
    for (int k = 0; k < 4; k++) { const uint32_t n = g * 4u + k; Av[k] = (live && n < a.N) ? a.A[(size_t)c * a.N + n] : 0.0f; }
    {
        float zs[4] = {0.0f, 0.0f, 0.0f, 0.0f}, q[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
        for (uint32_t t = t0; t < t1; t++) {
            const float dtc = STAGE ? dts[t * CH + x / LG] : (live ? dtp[(size_t)t * a.C + c] : 0.0f), dx = dtc * (STAGE ? xs[t * CH + x / LG] : (live ? xp[(size_t)t * a.C + c] : 0.0f));
            float Bv[4];
            load4(bcp + (size_t)t * a.ldb + a.b0, g * 4u, a.N, vec4, Bv);
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (g * 4u + k < a.N) { const float z = dtc * Av[k]; q[k] = decay_drive(z, q[k], dx * Bv[k]); zs[k] += z; }
        }
#pragma unroll
        for (int k = 0; k < 4; k++) { P[seg][x][k] = expf(zs[k]); Q[seg][x][k] = q[k]; }
    }
    __syncthreads();
    if (seg == 0 && live) {
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t n = g * 4u + k;
            if (n >= a.N) continue;
            float s = a.S[(size_t)c * a.N + n];
            for (uint32_t sg = 0; sg < nseg; sg++) { const float pg = P[sg][x][k], qg = Q[sg][x][k]; P[sg][x][k] = s; s = fmaf(pg, s, qg); }
            a.S[(size_t)c * a.N + n] = s;
        }
    }
    __syncthreads();
    float S[4];
#pragma unroll
    for (int k = 0; k < 4; k++) S[k] = (live && g * 4u + k < a.N) ? P[seg][x][k] : 0.0f;
    const float Dc = live ? a.Dv[c] : 0.0f;
#pragma unroll 4
    for (uint32_t t = t0; t < t1; t++) {
        const float dtc = STAGE ? dts[t * CH + x / LG] : (live ? dtp[(size_t)t * a.C + c] : 0.0f), xv = STAGE ? xs[t * CH + x / LG] : (live ? xp[(size_t)t * a.C + c] : 0.0f), dx = dtc * xv;
        const float *__restrict__ row = bcp + (size_t)t * a.ldb;
        float acc = 0.0f, Bv[4], Cv[4];
        load4(row + a.b0, g * 4u, a.N, vec4, Bv); load4(row + a.c0, g * 4u, a.N, vec4, Cv);
#pragma unroll
        for (int k = 0; k < 4; k++)
            if (g * 4u + k < a.N) { S[k] = decay_drive(dtc * Av[k], S[k], dx * Bv[k]); acc = fmaf(S[k], Cv[k], acc); }
#pragma unroll
        for (int off = LG / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (live && g == 0) yp[(size_t)t * a.C + c] = (acc + Dc * xv) * siluf_(STAGE ? zst[t * CH + x / LG] : zp[(size_t)t * a.ldz + c]);
    }
}

// PolyNorm over a token's feed-forward vector, in place: a N(z) + b N(z^2) + c N(z^3) + e with powers taken element by element
// and N(u) = u / sqrt(mean(u^2) + eps); coef = (a, b, c, e).  One block per token.
struct PolyArgs { float *z; uint32_t ld; const float *coef; uint32_t T, F; float eps; };
__global__ void __launch_bounds__(256) k_polynorm(const PolyArgs a) {
    pdl_enter();
    __shared__ float red[32];
    float *z = a.z + (size_t)blockIdx.x * a.ld;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (uint32_t i = threadIdx.x; i < a.F; i += blockDim.x) { const float v = z[i], v2 = v * v, v3 = v2 * v; s2 += v2; s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6); }
    s2 = block_sum(s2, red); s4 = block_sum(s4, red); s6 = block_sum(s6, red);
    const float r1 = a.coef[0] / sqrtf(s2 / (float)a.F + a.eps), r2 = a.coef[1] / sqrtf(s4 / (float)a.F + a.eps), r3 = a.coef[2] / sqrtf(s6 / (float)a.F + a.eps);
    const float e = a.coef[3];
    for (uint32_t i = threadIdx.x; i < a.F; i += blockDim.x) { const float v = z[i], v2 = v * v; z[i] = fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e))); }
}

}  // namespace lm
}  // namespace nb
