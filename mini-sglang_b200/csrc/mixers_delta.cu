// Kernels of softmax attention with a learned term in the denominator, of the gated delta rule and of the block
// arrangement with scaled sums and a per-layer token input (sm_100a; plain C entry points, loaded by ops.py as the
// library "mixers_delta", built only for models with such parts):
//
//   scaled_add_norm_kernel     res += x * s (s a float32 vector of the width), then y = rms(res) * w or y = res (or no y)
//   rotary_angles_kernel       cos | sin of position * frequency for the tokens of a step, in double precision
//   sink_qkv_prep_kernel       rotation of q and k heads in halves from the step's angles, values blended with another
//                              layer's, K and V rows (of head sizes of their own) into the paged cache
//   sink_attention_kernel      causal softmax attention within a window over the paged cache, scores capped by a tanh
//                              where asked, with exp(sink_h) in the denominator; float32 arithmetic, any head size to 512
//   sink_attention_mma_kernel  the same for bfloat16 with both products on mma.sync tiles (64 rows a block, float32 scores,
//                              running maximum and sum), prompts, portions and decoded tokens
//   sink_merge_kernel          one-token steps cut a request's keys into pieces for blocks of their own: the pieces'
//                              (max, sum, weighted values) are joined, in the order of the pieces, with the sink
//   delta_prep_kernel          unit-length q and k, beta and g of the gated delta rule from their projections, all tokens
//   delta_rule_kernel          S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per head, token by token
//   side_gate_mul_kernel       gelu_tanh(gate) times a slice of a per-token table's row
//
// Scores, weights, norms, angles, decays, states and everything that enters the recurrence are float32 (angles: double);
// T is the type of the activations between kernels (float or bfloat16).  Key chunks and pieces are anchored at absolute
// positions, so the order of a position's sums does not depend on how the tokens were cut into steps.
#include "common.cuh"
#include <math.h>

namespace {
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_tanhf_(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
}  // namespace

// ---------------------------------------------------------------------------------------
// res += x * s;  y = res / sqrt(mean(res^2) + eps) * w  (w given)  or  y = res  (y given, no w)
// One block per row; the sum of squares in float32.
// ---------------------------------------------------------------------------------------
template <typename A, typename O>
__global__ void __launch_bounds__(256) scaled_add_norm_kernel(const A* __restrict__ x, const float* __restrict__ s, float* __restrict__ res,
                                                              const float* __restrict__ w, float eps, O* __restrict__ y, int H) {
    __shared__ float scratch[32];
    const size_t row = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = fmaf(to_f32<A>(x[row + i]), s[i], res[row + i]);
        res[row + i] = v;
        ss = fmaf(v, v, ss);
    }
    if (y == nullptr) return;
    float rs = 1.f;
    if (w != nullptr) rs = 1.f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) y[row + i] = from_f32<O>(w ? res[row + i] * rs * w[i] : res[row + i]);
}

// The same with four neighbouring columns a thread and turn (H a multiple of 4, rows 16-byte aligned); the row's new values stay
// in registers between the sum and the norm where the row has at most 4 * NV * blockDim columns.
template <typename A, typename O, int NV>
__global__ void __launch_bounds__(256) scaled_add_norm_vec_kernel(const A* __restrict__ x, const float* __restrict__ s, float* __restrict__ res,
                                                                  const float* __restrict__ w, float eps, O* __restrict__ y, int H) {
    __shared__ float scratch[32];
    const size_t row = (size_t)blockIdx.x * H;
    float v[NV][4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        if (i < H) {
            const float4 r4 = *reinterpret_cast<const float4*>(res + row + i), s4 = *reinterpret_cast<const float4*>(s + i);
            float xv[4];
            if constexpr (sizeof(A) == 4) {
                const float4 x4 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + row + i);
                xv[0] = x4.x; xv[1] = x4.y; xv[2] = x4.z; xv[3] = x4.w;
            } else {
                const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(x) + row + i);
                xv[0] = __uint_as_float(u.x << 16); xv[1] = __uint_as_float(u.x & 0xffff0000u);
                xv[2] = __uint_as_float(u.y << 16); xv[3] = __uint_as_float(u.y & 0xffff0000u);
            }
            v[k][0] = fmaf(xv[0], s4.x, r4.x); v[k][1] = fmaf(xv[1], s4.y, r4.y);
            v[k][2] = fmaf(xv[2], s4.z, r4.z); v[k][3] = fmaf(xv[3], s4.w, r4.w);
            *reinterpret_cast<float4*>(res + row + i) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
            ss += v[k][0] * v[k][0] + v[k][1] * v[k][1] + v[k][2] * v[k][2] + v[k][3] * v[k][3];
        }
    }
    if (y == nullptr) return;
    float rs = 1.f;
    if (w != nullptr) rs = 1.f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        if (i < H) {
            float o[4];
            if (w != nullptr) {
                const float4 w4 = *reinterpret_cast<const float4*>(w + i);
                o[0] = v[k][0] * rs * w4.x; o[1] = v[k][1] * rs * w4.y; o[2] = v[k][2] * rs * w4.z; o[3] = v[k][3] * rs * w4.w;
            } else {
                o[0] = v[k][0]; o[1] = v[k][1]; o[2] = v[k][2]; o[3] = v[k][3];
            }
            if constexpr (sizeof(O) == 4) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + row + i) = make_float4(o[0], o[1], o[2], o[3]);
            } else {
                const __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + row + i) =
                    make_uint2(*reinterpret_cast<const unsigned*>(&a), *reinterpret_cast<const unsigned*>(&b));
            }
        }
    }
}

MSGL_API int msgl_scaled_add_norm(const void* x, int x_is_f32, const float* s, float* res, const float* w, float eps, void* y,
                                  int y_dtype, int T_, int H, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (H <= 0) return MSGL_ERR_SIZE;
    if (y_dtype != MSGL_F32 && y_dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const bool aligned = H % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)res % 16) == 0 && ((uintptr_t)s % 16) == 0 &&
                         ((uintptr_t)w % 16) == 0 && ((uintptr_t)y % 16) == 0 && (x_is_f32 || H % 8 == 0);
    if (aligned && H <= 4 * 4 * 256) {
        const int vt = H <= 1024 ? 64 : (H <= 4096 ? 256 : 256);
        const int nv = (H / 4 + vt - 1) / vt;
#define SANV(A, O, NV) scaled_add_norm_vec_kernel<A, O, NV><<<T_, vt, 0, stream>>>((const A*)x, s, res, w, eps, (O*)y, H)
#define SANV_T(NV)                                                                                                           \
    do {                                                                                                                     \
        if (y_dtype == MSGL_F32) { if (x_is_f32) SANV(float, float, NV); else SANV(__nv_bfloat16, float, NV); }              \
        else { if (x_is_f32) SANV(float, __nv_bfloat16, NV); else SANV(__nv_bfloat16, __nv_bfloat16, NV); }                  \
    } while (0)
        if (nv <= 1) SANV_T(1); else if (nv <= 2) SANV_T(2); else SANV_T(4);
#undef SANV_T
#undef SANV
        return msgl_check_launch();
    }
    const int threads = H >= 1024 ? 256 : 128;
#define SAN(A, O) scaled_add_norm_kernel<A, O><<<T_, threads, 0, stream>>>((const A*)x, s, res, w, eps, (O*)y, H)
    if (y_dtype == MSGL_F32) { if (x_is_f32) SAN(float, float); else SAN(__nv_bfloat16, float); }
    else if (y_dtype == MSGL_BF16) { if (x_is_f32) SAN(float, __nv_bfloat16); else SAN(__nv_bfloat16, __nv_bfloat16); }
    else return MSGL_ERR_DTYPE;
#undef SAN
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// out[t, i] = mag * cos(position_t * f_i),  out[t, half + i] = mag * sin(position_t * f_i),  i < half; double precision
// ---------------------------------------------------------------------------------------
__global__ void rotary_angles_kernel(const int* __restrict__ positions, const double* __restrict__ freq, double mag, float* __restrict__ out,
                                     int T_, int half) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T_ * half) return;
    const int t = idx / half, i = idx - t * half;
    double s, c;
    sincos((double)positions[t] * freq[i], &s, &c);
    out[(size_t)t * 2 * half + i] = (float)(c * mag);
    out[(size_t)t * 2 * half + half + i] = (float)(s * mag);
}

MSGL_API int msgl_rotary_angles(const int* positions, const double* freq, double mag, float* out, int T_, int half, cudaStream_t stream) {
    if (T_ <= 0 || half <= 0) return MSGL_OK;
    const int n = T_ * half;
    rotary_angles_kernel<<<(n + 127) / 128, 128, 0, stream>>>(positions, freq, mag, out, T_, half);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// q, k, v of a packed projection row [q: n_q * d | k: n_kv * d | v: n_kv * dv]:
//   q and k heads: the first `rot` elements turn in halves by the token's angles (cs [T][rot] = cos | sin), the rest pass
//   v heads: v <- (1 - lam) v + lam v_first where another layer's values are given
//   q -> q_out [T, n_q, d]; k, v -> the paged caches at token slot out_loc[t] (where given)
// One warp per (token, head of q, k or v).
// ---------------------------------------------------------------------------------------
struct SinkPrepParams {
    const void* proj; long long stride;
    const float* cs; int rot;
    const void* v_first; long long vf_stride; float lam;
    const int* out_loc; void* q_out; void* k_cache; void* v_cache;
    int page_size, n_q, n_kv, d, dv, T;
};

template <typename T>
__global__ void __launch_bounds__(128) sink_qkv_prep_kernel(const SinkPrepParams p) {
    const int t = blockIdx.x;
    const int slot = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int n_slots = p.n_q + 2 * p.n_kv;
    if (slot >= n_slots) return;
    const T* row = reinterpret_cast<const T*>(p.proj) + (size_t)t * p.stride;
    const int half = p.rot >> 1;
    const float* cs = p.cs ? p.cs + (size_t)t * p.rot : nullptr;
    if (slot < p.n_q + p.n_kv) {
        const bool is_q = slot < p.n_q;
        const int h = is_q ? slot : slot - p.n_q;
        const T* src = row + (is_q ? 0 : (size_t)p.n_q * p.d) + (size_t)h * p.d;
        T* dst;
        if (is_q) {
            dst = reinterpret_cast<T*>(p.q_out) + ((size_t)t * p.n_q + h) * p.d;
        } else {
            if (p.k_cache == nullptr) return;
            const int loc = p.out_loc[t];
            dst = reinterpret_cast<T*>(p.k_cache) + (((size_t)(loc / p.page_size) * p.n_kv + h) * p.page_size + loc % p.page_size) * p.d;
        }
        for (int e = lane; e < p.d; e += 32) {
            float v = to_f32<T>(src[e]);
            if (cs != nullptr && e < p.rot) {
                if (e < half) v = v * cs[e] - to_f32<T>(src[e + half]) * cs[half + e];
                else v = v * cs[e - half] + to_f32<T>(src[e - half]) * cs[e];
            }
            dst[e] = from_f32<T>(v);
        }
    } else {
        if (p.v_cache == nullptr) return;
        const int h = slot - p.n_q - p.n_kv;
        const T* src = row + (size_t)(p.n_q + p.n_kv) * p.d + (size_t)h * p.dv;
        const T* vf = p.v_first ? reinterpret_cast<const T*>(p.v_first) + (size_t)t * p.vf_stride + (size_t)h * p.dv : nullptr;
        const int loc = p.out_loc[t];
        T* dst = reinterpret_cast<T*>(p.v_cache) + (((size_t)(loc / p.page_size) * p.n_kv + h) * p.page_size + loc % p.page_size) * p.dv;
        for (int e = lane; e < p.dv; e += 32) {
            float v = to_f32<T>(src[e]);
            if (vf != nullptr) v = (1.f - p.lam) * v + p.lam * to_f32<T>(vf[e]);
            dst[e] = from_f32<T>(v);
        }
    }
}

MSGL_API int msgl_sink_qkv_prep(const void* proj, long long stride, const float* cs, int rot, const void* v_first, long long vf_stride,
                                float lam, const int* out_loc, void* q_out, void* k_cache, void* v_cache, int page_size, int n_q, int n_kv,
                                int d, int dv, int T_, int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (d <= 0 || dv <= 0 || n_q <= 0 || n_kv <= 0 || rot < 0 || rot > d || (rot & 1) || page_size < 1 || (rot > 0 && cs == nullptr) ||
        (k_cache != nullptr && (out_loc == nullptr || v_cache == nullptr)))
        return MSGL_ERR_SIZE;
    SinkPrepParams p;
    p.proj = proj; p.stride = stride; p.cs = rot > 0 ? cs : nullptr; p.rot = rot; p.v_first = v_first; p.vf_stride = vf_stride; p.lam = lam;
    p.out_loc = out_loc; p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache; p.page_size = page_size; p.n_q = n_q; p.n_kv = n_kv;
    p.d = d; p.dv = dv; p.T = T_;
    const dim3 grid(T_, (n_q + 2 * n_kv + 3) / 4);
    if (dtype == MSGL_F32) sink_qkv_prep_kernel<float><<<grid, 128, 0, stream>>>(p);
    else if (dtype == MSGL_BF16) sink_qkv_prep_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(p);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Causal softmax attention within a window over the paged cache, with a sink
//
//   s(i, j) = q[i, h] . k[j, g] * scale;   s <- cap * tanh(s / cap) (cap > 0);   j <= i and (no window or i - j < window)
//   o[i, h, :] = sum_j exp(s(i, j)) v[j, g, :] / (sum_j exp(s(i, j)) + exp(sink[h]))
//
// A block owns a tile of QT tokens x GH query heads of one kv head (SK_ROWS rows, one warp each) and walks the keys in
// chunks of 32 anchored at multiples of 32, with a running maximum and sum per row.  In the score phase lane l of a row's
// warp takes key l of the chunk, in the value phase lane l takes the output elements l, l + 32, ...  Cache rows behind the
// window of the tile's first token are never read (their pages may be gone).  With `splits` > 1 (steps in which every
// request brings one token) block z walks piece z of the request's keys, pieces of `split_keys` keys anchored at multiples
// of split_keys from the piece that holds the first key the token sees, and leaves (max, sum, weighted values) in `part`.
// ---------------------------------------------------------------------------------------
#define SK_ROWS 8
#define SK_KC 32
#define SK_MAX_DPL 16       // head sizes up to 512

struct SinkAttnParams {
    const void* q;            // [T, n_q, d]
    const void* k_cache; const void* v_cache;
    const int* q_start; const int* kv_len; const int* block_table; int bt_stride;
    int uniform;
    const float* sink;                            // [n_q]
    void* out; long long out_stride;              // [T rows][n_q * dv]
    float* part_o; float* part_ml; int splits, split_keys;      // [splits][T][n_q][dv], [splits][T][n_q][2]
    int T, B, n_q, n_kv, d, dv, page_size, QT, GH, window;
    float scale, softcap;
};

template <typename T, int DPL>
__global__ void __launch_bounds__(SK_ROWS * 32) sink_attention_kernel(const SinkAttnParams p) {
    extern __shared__ float smem[];
    const int d = p.d, dv = p.dv;
    float* qs = smem;                                // [SK_ROWS][d]
    float* ks = qs + SK_ROWS * d;                    // [SK_KC][d + 1]
    float* vs = ks + SK_KC * (d + 1);                // [SK_KC][dv]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ int tile_sh[2];
    int req, t0;
    if (p.uniform) {
        req = blockIdx.x; t0 = 0;
    } else {
        if (tid == 0) {
            int left = blockIdx.x, found = -1, at = 0;
            for (int r = 0; r < p.B; ++r) {
                const int nt = (p.q_start[r + 1] - p.q_start[r] + p.QT - 1) / p.QT;
                if (left < nt) { found = r; at = left * p.QT; break; }
                left -= nt;
            }
            tile_sh[0] = found; tile_sh[1] = at;
        }
        __syncthreads();
        req = tile_sh[0]; t0 = tile_sh[1];
    }
    if (req < 0 || req >= p.B) return;
    const int G = p.n_q / p.n_kv;
    const int n_chunks = (G + p.GH - 1) / p.GH;
    const int kvh = blockIdx.y / n_chunks, chunk = blockIdx.y - kvh * n_chunks;
    const int q_base = p.q_start[req], q_len = p.q_start[req + 1] - q_base, kv_len = p.kv_len[req];
    const int n_tok = min(p.QT, q_len - t0);
    if (n_tok <= 0) return;
    const int p_min = kv_len - q_len + t0, p_max = p_min + n_tok - 1;
    int key_lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0, key_hi = p_max + 1;      // keys this block walks: [key_lo, key_hi)
    if (p.splits > 1) {
        const int piece = key_lo / p.split_keys + blockIdx.z;
        key_lo = max(key_lo, piece * p.split_keys);
        key_hi = min(key_hi, (piece + 1) * p.split_keys);
    }

    const int tl = warp / p.GH, hl = warp - tl * p.GH;
    const int hg = chunk * p.GH + hl;
    const bool row_ok = tl < n_tok && hg < G && tl < p.QT;
    const int head = kvh * G + (row_ok ? hg : 0);
    const int tok = q_base + t0 + (row_ok ? tl : 0);
    const int pos = p_min + tl;
    const int first_seen = p.window > 0 ? pos - p.window + 1 : 0;
    const T* qg = reinterpret_cast<const T*>(p.q);
    for (int e = lane; e < d; e += 32) qs[warp * d + e] = row_ok ? to_f32<T>(qg[((size_t)tok * p.n_q + head) * d + e]) : 0.f;
    const T* kc = reinterpret_cast<const T*>(p.k_cache);
    const T* vc = reinterpret_cast<const T*>(p.v_cache);
    const int* bt = p.block_table + (size_t)req * p.bt_stride;
    const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;

    float o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    for (int key0 = key_lo - key_lo % SK_KC; key0 < key_hi; key0 += SK_KC) {
        __syncthreads();
        for (int idx = tid; idx < SK_KC * d; idx += SK_ROWS * 32) {
            const int kr = idx / d, e = idx - kr * d;
            const int key = key0 + kr;
            float kv = 0.f;
            if (key >= key_lo && key < key_hi) {
                const int page = bt[key / p.page_size];
                kv = to_f32<T>(kc[(((size_t)page * p.n_kv + kvh) * p.page_size + (key % p.page_size)) * d + e]);
            }
            ks[kr * (d + 1) + e] = kv;
        }
        for (int idx = tid; idx < SK_KC * dv; idx += SK_ROWS * 32) {
            const int kr = idx / dv, e = idx - kr * dv;
            const int key = key0 + kr;
            float vv = 0.f;
            if (key >= key_lo && key < key_hi) {
                const int page = bt[key / p.page_size];
                vv = to_f32<T>(vc[(((size_t)page * p.n_kv + kvh) * p.page_size + (key % p.page_size)) * dv + e]);
            }
            vs[kr * dv + e] = vv;
        }
        __syncthreads();
        const int key = key0 + lane;
        const bool vis = row_ok && key <= pos && key >= first_seen && key >= key_lo && key < key_hi;
        float sc = -INFINITY;
        if (vis) {
            float acc = 0.f;
            const float* qr = qs + warp * d;
            const float* kr = ks + lane * (d + 1);
            for (int e = 0; e < d; ++e) acc = fmaf(qr[e], kr[e], acc);
            sc = acc * p.scale;
            if (p.softcap > 0.f) sc = p.softcap * tanhf(sc * inv_cap);
        }
        const float cm = warp_max(sc);
        if (cm == -INFINITY) continue;                               // warp-uniform: no key of the chunk is seen by this row
        const float m_new = fmaxf(m_run, cm);
        const float corr = expf(m_run - m_new);                      // 0 at the first seen chunk (m_run = -inf)
        const float pr = vis ? expf(sc - m_new) : 0.f;
        l_run = l_run * corr + warp_sum(pr);
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] *= corr;
        for (int j = 0; j < SK_KC; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            if (pj == 0.f) continue;                                 // warp-uniform
            const float* vr = vs + j * dv;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int e = lane + 32 * i;
                if (e < dv) o[i] = fmaf(pj, vr[e], o[i]);
            }
        }
    }
    if (!row_ok) return;
    if (p.splits > 1) {
        const size_t r = ((size_t)blockIdx.z * p.T + tok) * p.n_q + head;
        float* pg = p.part_o + r * dv;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int e = lane + 32 * i;
            if (e < dv) pg[e] = o[i];
        }
        if (lane == 0) { p.part_ml[2 * r] = m_run; p.part_ml[2 * r + 1] = l_run; }
        return;
    }
    const float sk = p.sink[head];
    const float M = fmaxf(m_run, sk);
    const float f = expf(m_run - M);
    const float inv = f / (l_run * f + expf(sk - M));
    T* og = reinterpret_cast<T*>(p.out) + (size_t)tok * p.out_stride + (size_t)head * dv;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int e = lane + 32 * i;
        if (e < dv) og[e] = from_f32<T>(o[i] * inv);
    }
}

// the pieces of a one-token step joined, in the order of the pieces: one block per token, a thread per output element
template <typename T>
__global__ void __launch_bounds__(128) sink_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                         const float* __restrict__ sink, T* __restrict__ out, long long out_stride,
                                                         int T_, int n_q, int dv, int splits) {
    const int t = blockIdx.x, head = blockIdx.y;
    const size_t r0 = (size_t)t * n_q + head, step = (size_t)T_ * n_q;
    float M = sink[head];
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[2 * (r0 + s * step)]);
    float den = expf(sink[head] - M);
    for (int s = 0; s < splits; ++s) den = fmaf(part_ml[2 * (r0 + s * step) + 1], expf(part_ml[2 * (r0 + s * step)] - M), den);
    const float inv = 1.f / den;
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float f = expf(part_ml[2 * (r0 + s * step)] - M);
            if (f != 0.f) acc = fmaf(part_o[(r0 + s * step) * dv + e], f, acc);
        }
        out[(size_t)t * out_stride + (size_t)head * dv + e] = from_f32<T>(acc * inv);
    }
}

MSGL_API int msgl_sink_attention(const void* q, const void* k_cache, const void* v_cache, const int* q_start, const int* kv_len,
                                 const int* block_table, int bt_stride, int uniform, int n_tiles, const float* sink, void* out,
                                 long long out_stride, float* part_o, float* part_ml, int splits, int split_keys, int T_, int B, int n_q,
                                 int n_kv, int d, int dv, int page_size, int QT, int GH, int window, float scale, float softcap, int dtype,
                                 cudaStream_t stream) {
    if (n_tiles <= 0) return MSGL_OK;
    if (d <= 0 || dv <= 0 || dv > 32 * SK_MAX_DPL || d > 32 * SK_MAX_DPL || n_kv <= 0 || n_q % n_kv || QT < 1 || GH < 1 ||
        QT * GH > SK_ROWS || page_size < 1 || sink == nullptr || window < 0 || splits < 1 ||
        (splits > 1 && (!uniform || part_o == nullptr || part_ml == nullptr || split_keys < SK_KC || split_keys % SK_KC)))
        return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    SinkAttnParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
    p.bt_stride = bt_stride; p.uniform = uniform; p.sink = sink; p.out = out; p.out_stride = out_stride; p.part_o = part_o;
    p.part_ml = part_ml; p.splits = splits; p.split_keys = split_keys; p.T = T_; p.B = B; p.n_q = n_q; p.n_kv = n_kv; p.d = d; p.dv = dv;
    p.page_size = page_size; p.QT = QT; p.GH = GH; p.window = window; p.scale = scale; p.softcap = softcap;
    const int G = n_q / n_kv;
    const dim3 grid(n_tiles, n_kv * ((G + GH - 1) / GH), splits);
    const size_t smem = ((size_t)SK_ROWS * d + (size_t)SK_KC * (d + 1) + (size_t)SK_KC * dv) * sizeof(float);
    const int dpl = (dv + 31) / 32;
#define SK_LAUNCH(N)                                                                                                         \
    do {                                                                                                                     \
        static MsglOncePerDevice once;                                                                                       \
        if (smem > 48 * 1024 && once.due()) {                                                                                \
            cudaFuncSetAttribute(sink_attention_kernel<float, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);  \
            cudaFuncSetAttribute(sink_attention_kernel<__nv_bfloat16, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            once.mark();                                                                                                     \
        }                                                                                                                    \
        if (dtype == MSGL_F32) sink_attention_kernel<float, N><<<grid, SK_ROWS * 32, smem, stream>>>(p);                     \
        else sink_attention_kernel<__nv_bfloat16, N><<<grid, SK_ROWS * 32, smem, stream>>>(p);                               \
    } while (0)
    if (dpl <= 1) SK_LAUNCH(1);
    else if (dpl <= 2) SK_LAUNCH(2);
    else if (dpl <= 4) SK_LAUNCH(4);
    else if (dpl <= 8) SK_LAUNCH(8);
    else SK_LAUNCH(16);
#undef SK_LAUNCH
    int code = msgl_check_launch();
    if (code != MSGL_OK || splits <= 1) return code;
    const dim3 g2(T_, n_q);
    if (dtype == MSGL_F32) sink_merge_kernel<float><<<g2, 128, 0, stream>>>(part_o, part_ml, sink, (float*)out, out_stride, T_, n_q, dv, splits);
    else sink_merge_kernel<__nv_bfloat16><<<g2, 128, 0, stream>>>(part_o, part_ml, sink, (__nv_bfloat16*)out, out_stride, T_, n_q, dv, splits);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16): S = Q K^T and O += P V by mma.sync m16n8k16 with float32 accumulators;
// scores, cap, running maximum and sum in float32 between them, the weights rounded to bfloat16 only as the operand of the
// value product.  A block owns 64 rows = 64 / G tokens x the G query heads of one kv head (so a key tile serves all its
// heads) and walks the key tiles of 64 anchored at multiples of 64 from the one that holds the first key its first token
// sees, two tiles in flight (cp.async).  Cache rows before that key and after the last token are not read (zero in shared
// memory).  Exponentials are 2^x of scores in log2 units.  DK, DV: the head sizes rounded up to a size the kernel is built
// for; columns beyond d, dv are zero in shared memory.
// ---------------------------------------------------------------------------------------
namespace {
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16_u32(unsigned s, const void* gmem, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4_u32(unsigned (&r)[4], unsigned s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans_u32(unsigned (&r)[4], unsigned s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float ex2_(float x) {          // 2^x on the special-function unit (-inf gives 0)
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(x));
    return e;
}
// tanh(x) = 1 - 2 / (e^2x + 1), to about 1e-6 absolutely
__device__ __forceinline__ float fast_tanh(float x) { return 1.f - __fdividef(2.f, ex2_(2.8853900817779268f * x) + 1.f); }
}  // namespace

#define SKM_R 64            // rows of a block
#define SKM_KT 64           // keys of a tile
#define SKM_THREADS 128
#define LOG2E_F 1.4426950408889634f
#define LN2_F 0.6931471805599453f

template <int DK, int DV>
__global__ void __launch_bounds__(SKM_THREADS) sink_attention_mma_kernel(const SinkAttnParams p) {
    constexpr int LDK = DK + 8, LDV = DV + 8;           // padded rows (elements): ldmatrix without bank conflicts
    constexpr int NKB = SKM_KT / 8, NDB = DV / 8;
    constexpr int CHK = DK / 8, CHV = DV / 8;           // 16-byte pieces of a row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [64][LDK]
    __nv_bfloat16* KVs = Qs + SKM_R * LDK;                                          // [stage][K: 64 x LDK | V: 64 x LDV]
    __shared__ int tile_sh[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.n_q / p.n_kv;
    const int Gc = G <= SKM_R ? G : SKM_R;
    const int n_chunks = G <= SKM_R ? 1 : (G + SKM_R - 1) / SKM_R;
    const int QT = G <= SKM_R ? SKM_R / G : 1;
    const int kvh = blockIdx.y / n_chunks, chunk = blockIdx.y - kvh * n_chunks;
    if (tid == 0) {
        if (p.uniform) {
            tile_sh[0] = blockIdx.x; tile_sh[1] = 0;
        } else {
            int left = (int)gridDim.x - 1 - (int)blockIdx.x, found = -1, at = 0;      // heaviest tiles first
            for (int r = 0; r < p.B; ++r) {
                const int nt = (p.q_start[r + 1] - p.q_start[r] + QT - 1) / QT;
                if (left < nt) { found = r; at = left * QT; break; }
                left -= nt;
            }
            tile_sh[0] = found; tile_sh[1] = at;
        }
    }
    __syncthreads();
    const int req = tile_sh[0], t0 = tile_sh[1];
    if (req < 0 || req >= p.B) return;
    const int q_base = p.q_start[req], q_len = p.q_start[req + 1] - q_base, kv_len = p.kv_len[req];
    const int n_tok = min(QT, q_len - t0);
    if (n_tok <= 0) return;
    const int p_min = kv_len - q_len + t0, p_max = p_min + n_tok - 1;
    const int key_lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;      // the first key any row of the block sees
    int kt_lo = key_lo / SKM_KT, kt_hi = p_max / SKM_KT + 1;
    if (p.splits > 1) {       // a piece is a whole number of tiles, counted from the piece that holds key_lo
        const int piece = key_lo / p.split_keys + (int)blockIdx.z;
        kt_lo = max(kt_lo, piece * (p.split_keys / SKM_KT));
        kt_hi = min(kt_hi, (piece + 1) * (p.split_keys / SKM_KT));
    }
    const int d = p.d, dv = p.dv;
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(p.k_cache);
    const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(p.v_cache);
    const int* bt = p.block_table + (size_t)req * p.bt_stride;
    const unsigned q_s = smem_u32(Qs), kv_s = smem_u32(KVs);
    constexpr unsigned K_BYTES = SKM_KT * LDK * 2u, STAGE_BYTES = K_BYTES + SKM_KT * LDV * 2u;

    const int row_base = warp * 16;
    const int r_lo = row_base + (lane >> 2), r_hi = r_lo + 8;
    const int tl_lo = r_lo / Gc, tl_hi = r_hi / Gc;
    const int hl_lo = r_lo - tl_lo * Gc, hl_hi = r_hi - tl_hi * Gc;
    const int pos_lo = p_min + tl_lo, pos_hi = p_min + tl_hi;
    const int first_lo = p.window > 0 ? pos_lo - p.window + 1 : 0, first_hi = p.window > 0 ? pos_hi - p.window + 1 : 0;
    float o[NDB][4];
#pragma unroll
    for (int i = 0; i < NDB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};       // log2 units; l: this thread's share of the row's sum

    if (kt_lo < kt_hi) {
        // ---- the block's query rows (zero where the tile has no token or head, and beyond d)
        for (int idx = tid; idx < SKM_R * CHK; idx += SKM_THREADS) {
            const int r = idx / CHK, c = idx - r * CHK;
            const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * SKM_R + hl;
            const bool valid = tl < n_tok && tl < QT && hg < G && c * 8 < d;
            const size_t tok = (size_t)(q_base + t0 + (valid ? tl : 0));
            const __nv_bfloat16* src = qg + (tok * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * d + (valid ? c * 8 : 0);
            cp_async16_u32(q_s + (unsigned)(r * LDK + c * 8) * 2u, src, valid);
        }
        // a thread copies half a row of K and of V per tile: row tid / 2, every second 16-byte piece
        const int ld_row = tid >> 1, ld_half = tid & 1;
        auto load_kv = [&](int stage, int kt) {
            const int key = kt * SKM_KT + ld_row;
            const bool live = key <= p_max && key >= key_lo;
            size_t row = 0;
            if (live) row = ((size_t)bt[key / p.page_size] * p.n_kv + kvh) * p.page_size + (key % p.page_size);
            const unsigned ks = kv_s + (unsigned)stage * STAGE_BYTES + (unsigned)(ld_row * LDK) * 2u;
            const unsigned vs = kv_s + (unsigned)stage * STAGE_BYTES + K_BYTES + (unsigned)(ld_row * LDV) * 2u;
#pragma unroll
            for (int c = ld_half; c < CHK; c += 2) {
                const bool ok = live && c * 8 < d;
                cp_async16_u32(ks + c * 16, kc + row * d + (ok ? c * 8 : 0), ok);
            }
#pragma unroll
            for (int c = ld_half; c < CHV; c += 2) {
                const bool ok = live && c * 8 < dv;
                cp_async16_u32(vs + c * 16, vc + row * dv + (ok ? c * 8 : 0), ok);
            }
        };
        load_kv(0, kt_lo);
        cp_async_commit();

        const bool warp_live = row_base / Gc < n_tok;       // else all 16 rows of the warp are empty: it copies, but multiplies nothing
        const int warp_pos_lo = p_min + row_base / Gc, warp_pos_hi = p_min + (row_base + 15) / Gc;
        const unsigned q_a = q_s + (unsigned)((row_base + (lane & 15)) * LDK + (lane >> 4) * 8) * 2u;
        const unsigned k_lane = (unsigned)(((lane & 7) + ((lane >> 4) & 1) * 8) * LDK + ((lane >> 3) & 1) * 8) * 2u;
        const unsigned v_lane = (unsigned)(((lane & 7) + ((lane >> 3) & 1) * 8) * LDV + ((lane >> 4) & 1) * 8) * 2u;
        const float scale2 = p.scale * LOG2E_F;
        const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f, cap2 = p.softcap * LOG2E_F;

        for (int kt = kt_lo; kt < kt_hi; ++kt) {
            const int stage = (kt - kt_lo) & 1;
            if (kt + 1 < kt_hi) {
                load_kv(stage ^ 1, kt + 1);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            const int key0 = kt * SKM_KT;
            // no row of the warp sees a key of this tile: the tile lies behind its last token or before its first token's window
            if (!warp_live || key0 > warp_pos_hi || (p.window > 0 && key0 + SKM_KT - 1 < warp_pos_lo - p.window + 1)) {
                __syncthreads();
                continue;
            }
            const unsigned ks_a = kv_s + (unsigned)stage * STAGE_BYTES + k_lane;
            const unsigned vs_a = kv_s + (unsigned)stage * STAGE_BYTES + K_BYTES + v_lane;

            float s[NKB][4];
#pragma unroll
            for (int i = 0; i < NKB; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk) {
                unsigned a[4];
                ldmatrix_x4_u32(a, q_a + kk * 32);
#pragma unroll
                for (int nb2 = 0; nb2 < NKB / 2; ++nb2) {
                    unsigned b[4];
                    ldmatrix_x4_u32(b, ks_a + (unsigned)(nb2 * 16 * LDK + kk * 16) * 2u);
                    mma_bf16_16816(s[2 * nb2], a, b[0], b[1]);
                    mma_bf16_16816(s[2 * nb2 + 1], a, b[2], b[3]);
                }
            }
            // ---- scores in log2 units, capped, masked; the tile's maximum per row
            const bool need_mask = key0 + SKM_KT - 1 > warp_pos_lo || (p.window > 0 && key0 < warp_pos_hi - p.window + 1);
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < NKB; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[nb][e] * scale2;
                    if (p.softcap > 0.f) v = cap2 * fast_tanh(s[nb][e] * p.scale * inv_cap);
                    if (need_mask) {
                        const int key = key0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                        const int pos = (e < 2) ? pos_lo : pos_hi, first = (e < 2) ? first_lo : first_hi;
                        if (key > pos || key < first) v = -INFINITY;
                    }
                    s[nb][e] = v;
                    tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
                }
            }
            float corr[2], m_use[2];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                float t = tmax[hf];
                t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 1));
                t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 2));
                const float m_new = fmaxf(m_run[hf], t);
                m_use[hf] = m_new == -INFINITY ? 0.f : m_new;            // a row that has seen no key yet: all weights 0
                corr[hf] = ex2_(m_run[hf] - m_use[hf]);                  // m_run = -inf gives 0
                m_run[hf] = m_new;
                l_run[hf] *= corr[hf];
            }
#pragma unroll
            for (int nb = 0; nb < NKB; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float w = ex2_(s[nb][e] - m_use[e >> 1]);
                    s[nb][e] = w;
                    l_run[e >> 1] += w;
                }
            }
#pragma unroll
            for (int nd = 0; nd < NDB; ++nd) { o[nd][0] *= corr[0]; o[nd][1] *= corr[0]; o[nd][2] *= corr[1]; o[nd][3] *= corr[1]; }
            // ---- O += P V
#pragma unroll
            for (int j = 0; j < NKB / 2; ++j) {
                unsigned a[4];
                a[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
                a[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
                a[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
                a[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
                for (int nd2 = 0; nd2 < DV / 16; ++nd2) {
                    unsigned b[4];
                    ldmatrix_x4_trans_u32(b, vs_a + (unsigned)(j * 16 * LDV + nd2 * 16) * 2u);
                    mma_bf16_16816(o[2 * nd2], a, b[0], b[1]);
                    mma_bf16_16816(o[2 * nd2 + 1], a, b[2], b[3]);
                }
            }
            __syncthreads();
        }
        cp_async_wait<0>();
    }

    __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int tl = half ? tl_hi : tl_lo, hl = half ? hl_hi : hl_lo, hg = chunk * SKM_R + hl;
        float l = l_run[half];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (!(tl < n_tok && tl < QT && hg < G)) continue;
        const int head = kvh * G + hg;
        const size_t tok = (size_t)(q_base + t0 + tl);
        if (p.splits > 1) {
            const size_t r = ((size_t)blockIdx.z * p.T + tok) * p.n_q + head;
            float* pg = p.part_o + r * dv;
#pragma unroll
            for (int nd = 0; nd < NDB; ++nd) {
                const int col = nd * 8 + (lane & 3) * 2;
                if (col < dv) *reinterpret_cast<float2*>(pg + col) = make_float2(o[nd][half * 2], o[nd][half * 2 + 1]);
            }
            if ((lane & 3) == 0) { p.part_ml[2 * r] = m_run[half] * LN2_F; p.part_ml[2 * r + 1] = l; }
            continue;
        }
        const float sk2 = p.sink[head] * LOG2E_F;
        const float M = fmaxf(m_run[half], sk2);
        const float f = ex2_(m_run[half] - M);
        const float inv = __fdividef(f, l * f + ex2_(sk2 - M));
        __nv_bfloat16* dst = og + tok * p.out_stride + (size_t)head * dv;
#pragma unroll
        for (int nd = 0; nd < NDB; ++nd) {
            const int col = nd * 8 + (lane & 3) * 2;
            if (col < dv)           // dv is a multiple of 8: a pair lies inside the row or outside it
                *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[nd][half * 2] * inv, o[nd][half * 2 + 1] * inv);
        }
    }
}

// The tensor-core launch: bfloat16, head sizes that are multiples of 8 up to 128, rows of `out` that pairs of elements can be
// stored into.  n_tiles: the sum over the requests of ceil(tokens / QT) with QT = 64 / (heads per kv head) (1 beyond 64), or
// with `uniform` (every request brings one token) the number of requests; then `splits` pieces of `split_keys` keys (a
// multiple of 64) go to blocks of their own, which leave (max, sum, weighted values) for sink_merge_kernel.
MSGL_API int msgl_sink_attention_mma(const void* q, const void* k_cache, const void* v_cache, const int* q_start, const int* kv_len,
                                     const int* block_table, int bt_stride, int uniform, int n_tiles, const float* sink, void* out,
                                     long long out_stride, float* part_o, float* part_ml, int splits, int split_keys, int T_, int B, int n_q,
                                     int n_kv, int d, int dv, int page_size, int window, float scale, float softcap, cudaStream_t stream) {
    if (n_tiles <= 0) return MSGL_OK;
    if (d <= 0 || dv <= 0 || d > 128 || dv > 128 || d % 8 || dv % 8 || n_kv <= 0 || n_q % n_kv || page_size < 1 || sink == nullptr ||
        window < 0 || (out_stride & 1) || ((size_t)out & 3) || splits < 1 ||
        (splits > 1 && (!uniform || part_o == nullptr || part_ml == nullptr || split_keys < SKM_KT || split_keys % SKM_KT || ((size_t)part_o & 7))))
        return MSGL_ERR_SIZE;
    SinkAttnParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
    p.bt_stride = bt_stride; p.uniform = uniform; p.sink = sink; p.out = out; p.out_stride = out_stride; p.part_o = part_o;
    p.part_ml = part_ml; p.splits = splits; p.split_keys = split_keys; p.T = T_; p.B = B; p.n_q = n_q; p.n_kv = n_kv; p.d = d; p.dv = dv;
    p.page_size = page_size; p.QT = 0; p.GH = 0; p.window = window; p.scale = scale; p.softcap = softcap;
    const int G = n_q / n_kv;
    const dim3 grid(n_tiles, n_kv * (G <= SKM_R ? 1 : (G + SKM_R - 1) / SKM_R), splits);
#define SKM_LAUNCH(DK, DV)                                                                                                   \
    do {                                                                                                                     \
        const size_t smem = ((size_t)SKM_R * (DK + 8) + 2 * ((size_t)SKM_KT * (DK + 8) + (size_t)SKM_KT * (DV + 8))) * 2;    \
        static MsglOncePerDevice once;                                                                                       \
        if (once.due()) {                                                                                                    \
            cudaFuncSetAttribute(sink_attention_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            once.mark();                                                                                                     \
        }                                                                                                                    \
        sink_attention_mma_kernel<DK, DV><<<grid, SKM_THREADS, smem, stream>>>(p);                                           \
    } while (0)
#define SKM_BY_DV(DK)                                                                                                        \
    do {                                                                                                                     \
        if (dv <= 64) SKM_LAUNCH(DK, 64);                                                                                    \
        else if (dv <= 96) SKM_LAUNCH(DK, 96);                                                                               \
        else SKM_LAUNCH(DK, 128);                                                                                            \
    } while (0)
    if (d <= 64) SKM_BY_DV(64);
    else if (d <= 96) SKM_BY_DV(96);
    else SKM_BY_DV(128);
#undef SKM_BY_DV
#undef SKM_LAUNCH
    int code = msgl_check_launch();
    if (code != MSGL_OK || splits <= 1) return code;
    const dim3 g2(T_, n_q);
    sink_merge_kernel<__nv_bfloat16><<<g2, 128, 0, stream>>>(part_o, part_ml, sink, (__nv_bfloat16*)out, out_stride, T_, n_q, dv, splits);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// The gated delta rule, token by token
//
//   per head h (q/k head g = h / (heads / kv_heads)), state S [d][dv] float32 per request, per token t:
//     qn = q / sqrt(sum q^2 + 1e-6) * d^-1/2,  kn = k / sqrt(sum k^2 + 1e-6)
//     beta = sigmoid(pb[t, h]);  g = exp(-exp(A_log[h]) * softplus(pa[t, h] + dt_bias[h]))
//     S <- g S;  u = beta (v - S^T kn);  S <- S + kn u^T;  o[t, h, :] = S^T qn
//   qkv row [T][kv_heads * d | kv_heads * d | heads * dv] (what the convolution left); pa, pb column ranges of the packed
//   projection.
// delta_prep_kernel makes what does not depend on the state, all tokens side by side: (kn, qn) pairs [T][kv_heads][d] and
// (beta, g, kn . qn) [T][heads], float32.  delta_rule_kernel then walks a request's tokens in order.  The columns of a state
// do not meet: a warp owns DR_WCOLS columns of one (request, head) state, DR_PARTS lanes share a column's rows (each keeps its
// RPT rows in registers), and a token costs the warp two shuffle rounds and no barrier.  Both products with the old state are
// taken in one pass, A = S^T kn and Q = S^T qn, and o = g Q + (kn . qn) u.  The tokens go through shared memory in batches
// of DR_TB, the next batch on its way (cp.async; the block's columns of v through registers) while the current one is walked:
// a barrier a batch.  Few columns in all (one request's prompt): blocks of DR_FEW_WARPS warps, so that more SMs take part;
// else DR_MANY_WARPS.
// ---------------------------------------------------------------------------------------
#define DR_WCOLS 4
#define DR_PARTS 8
#ifndef DR_TB
#define DR_TB 16
#endif
#ifndef DR_FEW_WARPS
#define DR_FEW_WARPS 4
#endif
#ifndef DR_MANY_WARPS
#define DR_MANY_WARPS 8
#endif

struct DeltaParams {
    const void* qkv; const void* proj; long long proj_stride; int a_off, b_off;
    const float* a_log; const float* dt_bias;
    float2* kq; float4* sc;                      // what delta_prep_kernel leaves
    float* state; const int* q_start; const int* slots; float* out;
    int heads, kv_heads, d, dv, T;
};

template <typename T>
__global__ void __launch_bounds__(128) delta_prep_kernel(const DeltaParams p) {
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int g = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (g >= p.kv_heads) return;
    const int d = p.d, Ck = p.kv_heads * d, W = 2 * Ck + p.heads * p.dv;
    const T* rowp = reinterpret_cast<const T*>(p.qkv) + (size_t)t * W;
    float sq = 0.f, sk = 0.f;
    for (int e = lane; e < d; e += 32) {
        const float qe = to_f32<T>(rowp[(size_t)g * d + e]), ke = to_f32<T>(rowp[Ck + (size_t)g * d + e]);
        sq = fmaf(qe, qe, sq); sk = fmaf(ke, ke, sk);
    }
    sq = warp_sum(sq); sk = warp_sum(sk);
    const float rq = (1.f / sqrtf((float)d)) / sqrtf(sq + 1e-6f), rk = 1.f / sqrtf(sk + 1e-6f);
    float2* dst = p.kq + ((size_t)t * p.kv_heads + g) * d;
    float dot = 0.f;
    for (int e = lane; e < d; e += 32) {
        const float qe = to_f32<T>(rowp[(size_t)g * d + e]) * rq, ke = to_f32<T>(rowp[Ck + (size_t)g * d + e]) * rk;
        dst[e] = make_float2(ke, qe);
        dot = fmaf(ke, qe, dot);
    }
    dot = warp_sum(dot);
    const int per = p.heads / p.kv_heads;
    const T* proj = reinterpret_cast<const T*>(p.proj) + (size_t)t * p.proj_stride;
    for (int i = lane; i < per; i += 32) {
        const int h = g * per + i;
        const float pa = to_f32<T>(proj[p.a_off + h]), pb = to_f32<T>(proj[p.b_off + h]);
        p.sc[(size_t)t * p.heads + h] = make_float4(sigmoidf_(pb), expf(-expf(p.a_log[h]) * softplusf_(pa + p.dt_bias[h])), dot, 0.f);
    }
}

namespace {
__device__ __forceinline__ void cp_async8_(void* smem_dst, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(gmem));
}
__device__ __forceinline__ void cp_async16_(void* smem_dst, const void* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(gmem));
}
}  // namespace

template <typename T, int RPT, bool EXACT /* d == RPT * DR_PARTS: no row of a thread lies beyond the state */>
__global__ void __launch_bounds__(DR_MANY_WARPS * 32) delta_rule_kernel(const DeltaParams p) {
    extern __shared__ __align__(16) unsigned char dr_smem[];
    const int d = p.d, dv = p.dv;
    const int warps = blockDim.x >> 5, cols = warps * DR_WCOLS;
    constexpr int VPT = DR_TB * DR_WCOLS / 32;                          // values of v a thread brings per batch
    // per stage: sc [DR_TB] float4 | kq [DR_TB][d] float2 | v [DR_TB][cols] float
    const size_t stage_bytes = (size_t)DR_TB * 16 + (size_t)DR_TB * d * 8 + (size_t)DR_TB * cols * 4;
    const int h = blockIdx.x, r = blockIdx.y, c0 = blockIdx.z * cols;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = lane / DR_WCOLS, wc = lane % DR_WCOLS;             // lanes of a part read neighbouring columns
    const int g = h / (p.heads / p.kv_heads);
    const int t0 = p.q_start[r], n = p.q_start[r + 1] - t0;
    if (n <= 0) return;
    const int lcol = warp * DR_WCOLS + wc, col = c0 + lcol;
    const bool col_ok = col < dv;
    const int Ck = p.kv_heads * d, W = 2 * Ck + p.heads * dv;
    float* S = p.state + ((size_t)p.slots[r] * p.heads + h) * d * dv;
    float s_reg[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = part + DR_PARTS * i;
        s_reg[i] = ((EXACT || row < d) && col_ok) ? S[(size_t)row * dv + col] : 0.f;
    }
    const T* qkv = reinterpret_cast<const T*>(p.qkv);
    auto stage_sc = [&](int st) { return reinterpret_cast<float4*>(dr_smem + st * stage_bytes); };
    auto stage_kq = [&](int st) { return reinterpret_cast<float2*>(dr_smem + st * stage_bytes + DR_TB * 16); };
    auto stage_v = [&](int st) { return reinterpret_cast<float*>(dr_smem + st * stage_bytes + DR_TB * 16 + (size_t)DR_TB * d * 8); };
    auto issue = [&](int st, int b0) {           // the batch's (kn, qn) and (beta, g, kn . qn) on their way into a stage
        const int nb = min(DR_TB, n - b0);
        float2* kq = stage_kq(st);
        for (int j = 0; j < nb; ++j) {
            const float2* src = p.kq + ((size_t)(t0 + b0 + j) * p.kv_heads + g) * d;
            for (int e = tid; e < d; e += blockDim.x) cp_async8_(kq + j * d + e, src + e);
        }
        if (tid < nb) cp_async16_(stage_sc(st) + tid, p.sc + (size_t)(t0 + b0 + tid) * p.heads + h);
        asm volatile("cp.async.commit_group;\n" ::);
    };
    float vreg[VPT];
    const int vj = tid / cols, vc = tid - vj * cols, vstep = blockDim.x / cols;      // VPT * vstep = DR_TB
    auto load_v = [&](int b0) {                  // this block's columns of the batch's v into registers
        const int nb = min(DR_TB, n - b0);
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int j = vj + k * vstep;
            vreg[k] = (j < nb && c0 + vc < dv) ? to_f32<T>(qkv[(size_t)(t0 + b0 + j) * W + 2 * Ck + (size_t)h * dv + c0 + vc]) : 0.f;
        }
    };
    issue(0, 0);
    load_v(0);
    for (int b0 = 0, st = 0; b0 < n; b0 += DR_TB, st ^= 1) {
        const int nb = min(DR_TB, n - b0);
        float* vv = stage_v(st);
#pragma unroll
        for (int k = 0; k < VPT; ++k) vv[(vj + k * vstep) * cols + vc] = vreg[k];
        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();                         // the batch lies in its stage; the other stage is no longer read
        if (b0 + DR_TB < n) {
            issue(st ^ 1, b0 + DR_TB);
            load_v(b0 + DR_TB);
        }
        const float2* kq = stage_kq(st) + part;
        const float4* sc = stage_sc(st);
        for (int j = 0; j < nb; ++j) {
            const float2* kqj = kq + j * d;
            float2 kr[RPT];                      // the thread's rows of (kn, qn): read once, used by both passes
            float A0 = 0.f, A1 = 0.f, Q0 = 0.f, Q1 = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                kr[i] = (EXACT || part + DR_PARTS * i < d) ? kqj[DR_PARTS * i] : make_float2(0.f, 0.f);
                if (i & 1) { A1 = fmaf(s_reg[i], kr[i].x, A1); Q1 = fmaf(s_reg[i], kr[i].y, Q1); }
                else { A0 = fmaf(s_reg[i], kr[i].x, A0); Q0 = fmaf(s_reg[i], kr[i].y, Q0); }
            }
            float A = A0 + A1, Q = Q0 + Q1;
#pragma unroll
            for (int o = DR_WCOLS; o < 32; o <<= 1) {
                A += __shfl_xor_sync(0xffffffffu, A, o);
                Q += __shfl_xor_sync(0xffffffffu, Q, o);
            }
            const float4 c4 = sc[j];             // beta, g, kn . qn
            const float u = c4.x * (vv[j * cols + lcol] - c4.y * A);
#pragma unroll
            for (int i = 0; i < RPT; ++i) s_reg[i] = fmaf(kr[i].x, u, c4.y * s_reg[i]);
            if (part == 0 && col_ok) p.out[((size_t)(t0 + b0 + j) * p.heads + h) * dv + col] = fmaf(c4.z, u, c4.y * Q);
        }
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = part + DR_PARTS * i;
        if ((EXACT || row < d) && col_ok) S[(size_t)row * dv + col] = s_reg[i];
    }
}

// floats of scratch memory that msgl_delta_rule wants for T tokens
MSGL_API long long msgl_delta_rule_scratch(int T_, int heads, int kv_heads, int d) {
    return (long long)T_ * kv_heads * d * 2 + (long long)T_ * heads * 4;
}

MSGL_API int msgl_delta_rule(const void* qkv, const void* proj, long long proj_stride, int a_off, int b_off, const float* a_log,
                             const float* dt_bias, float* state, const int* q_start, const int* slots, float* out, float* scratch,
                             int heads, int kv_heads, int d, int dv, int T_, int B, int dtype, cudaStream_t stream) {
    if (B <= 0 || T_ <= 0) return MSGL_OK;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || d <= 0 || dv <= 0 || d > DR_PARTS * 64 || scratch == nullptr) return MSGL_ERR_SIZE;
    if (((uintptr_t)scratch & 15) != 0) return MSGL_ERR_ALIGN;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    DeltaParams p;
    p.qkv = qkv; p.proj = proj; p.proj_stride = proj_stride; p.a_off = a_off; p.b_off = b_off; p.a_log = a_log; p.dt_bias = dt_bias;
    p.sc = reinterpret_cast<float4*>(scratch);                                  // [T][heads] first: 16-byte rows stay aligned
    p.kq = reinterpret_cast<float2*>(scratch + (size_t)T_ * heads * 4);
    p.state = state; p.q_start = q_start; p.slots = slots; p.out = out; p.heads = heads; p.kv_heads = kv_heads; p.d = d; p.dv = dv; p.T = T_;
    const dim3 g0(T_, (kv_heads + 3) / 4);
    if (dtype == MSGL_F32) delta_prep_kernel<float><<<g0, 128, 0, stream>>>(p);
    else delta_prep_kernel<__nv_bfloat16><<<g0, 128, 0, stream>>>(p);
    int code = msgl_check_launch();
    if (code != MSGL_OK) return code;
    const int many_cols = DR_MANY_WARPS * DR_WCOLS;
    const long long blocks_many = (long long)heads * B * ((dv + many_cols - 1) / many_cols);
    const int warps = blocks_many >= 2LL * msgl_sm_count() ? DR_MANY_WARPS : DR_FEW_WARPS;
    const int cols = warps * DR_WCOLS;
    const dim3 grid(heads, B, (dv + cols - 1) / cols);
    const size_t smem = 2 * ((size_t)DR_TB * 16 + (size_t)DR_TB * d * 8 + (size_t)DR_TB * cols * 4);
    const int rpt = (d + DR_PARTS - 1) / DR_PARTS;
#define DR_LAUNCH_E(N, E)                                                                                                   \
    do {                                                                                                                    \
        static MsglOncePerDevice once;                                                                                      \
        if (smem > 48 * 1024 && once.due()) {                                                                               \
            cudaFuncSetAttribute(delta_rule_kernel<float, N, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);  \
            cudaFuncSetAttribute(delta_rule_kernel<__nv_bfloat16, N, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); \
            once.mark();                                                                                                    \
        }                                                                                                                   \
        if (dtype == MSGL_F32) delta_rule_kernel<float, N, E><<<grid, warps * 32, smem, stream>>>(p);                       \
        else delta_rule_kernel<__nv_bfloat16, N, E><<<grid, warps * 32, smem, stream>>>(p);                                 \
    } while (0)
#define DR_LAUNCH(N)                                                                                                        \
    do {                                                                                                                    \
        if (d == N * DR_PARTS) DR_LAUNCH_E(N, true); else DR_LAUNCH_E(N, false);                                            \
    } while (0)
    if (rpt <= 4) DR_LAUNCH(4);
    else if (rpt <= 8) DR_LAUNCH(8);
    else if (rpt <= 16) DR_LAUNCH(16);
    else if (rpt <= 32) DR_LAUNCH(32);
    else DR_LAUNCH(64);
#undef DR_LAUNCH
#undef DR_LAUNCH_E
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// out[t, j] = gelu_tanh(gate[t, j]) * table[ids[t]][offset + j],  j < dim: a layer's slice of a per-token table, gated
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void side_gate_mul_kernel(const T* __restrict__ gate, long long gate_stride, const T* __restrict__ table, int columns, int offset,
                                     const int* __restrict__ ids, int vocab, T* __restrict__ out, int dim, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / dim;
    const int j = (int)(i - t * dim);
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const float e = to_f32<T>(table[(size_t)id * columns + offset + j]);
    out[i] = from_f32<T>(gelu_tanhf_(to_f32<T>(gate[t * gate_stride + j])) * e);
}

MSGL_API int msgl_side_gate_mul(const void* gate, long long gate_stride, const void* table, int columns, int offset, const int* ids,
                                int vocab, void* out, int dim, int T_, int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (dim <= 0 || offset < 0 || offset + dim > columns || vocab <= 0) return MSGL_ERR_SIZE;
    const long long n = (long long)T_ * dim;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == MSGL_F32) side_gate_mul_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate, gate_stride, (const float*)table, columns, offset, ids, vocab, (float*)out, dim, n);
    else if (dtype == MSGL_BF16) side_gate_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate, gate_stride, (const __nv_bfloat16*)table, columns, offset, ids, vocab, (__nv_bfloat16*)out, dim, n);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}
