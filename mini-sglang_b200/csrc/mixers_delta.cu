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
//   sink_merge_kernel          one-token steps cut a request's keys into pieces for blocks of their own: the pieces'
//                              (max, sum, weighted values) are joined, in the order of the pieces, with the sink
//   delta_rule_kernel          S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per head, token by token, with
//                              unit-length q and k, beta and g made from their projections
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

MSGL_API int msgl_scaled_add_norm(const void* x, int x_is_f32, const float* s, float* res, const float* w, float eps, void* y,
                                  int y_dtype, int T_, int H, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (H <= 0) return MSGL_ERR_SIZE;
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
// The gated delta rule, token by token
//
//   per head h (q/k head g = h / (heads / kv_heads)), state S [d][dv] float32 per request, per token t:
//     qn = q / sqrt(sum q^2 + 1e-6) * d^-1/2,  kn = k / sqrt(sum k^2 + 1e-6)
//     beta = sigmoid(pb[t, h]);  g = exp(-exp(A_log[h]) * softplus(pa[t, h] + dt_bias[h]))
//     S <- g S;  u = beta (v - S^T kn);  S <- S + kn u^T;  o[t, h, :] = S^T qn
//   qkv row [T][kv_heads * d | kv_heads * d | heads * dv] (what the convolution left); pa, pb column ranges of the packed
//   projection.
// A block owns DR_COLS columns of one (request, head) state and walks the request's tokens in order; DR_PARTS warps share a
// column's rows, each thread keeps its RPT rows of the column in registers.  Both products with the old state are taken in
// one pass, A = S^T kn and Q = S^T qn, and o = g Q + (kn . qn) u, so a token costs one exchange between the warps.
// Tokens go through shared memory in batches of DR_TB with their norms, beta and g made on the way.
// ---------------------------------------------------------------------------------------
#define DR_COLS 32
#define DR_PARTS 8
#define DR_TB 8

struct DeltaParams {
    const void* qkv; const void* proj; long long proj_stride; int a_off, b_off;
    const float* a_log; const float* dt_bias;
    float* state; const int* q_start; const int* slots; float* out;
    int heads, kv_heads, d, dv;
};

template <typename T, int RPT>
__global__ void __launch_bounds__(DR_COLS * DR_PARTS) delta_rule_kernel(const DeltaParams p) {
    extern __shared__ float smem[];
    const int d = p.d, dv = p.dv;
    float2* kq = reinterpret_cast<float2*>(smem);                      // [DR_TB][d]: (kn, qn)
    float* vv = smem + 2 * DR_TB * d;                                  // [DR_TB][DR_COLS]
    float* sc = vv + DR_TB * DR_COLS;                                  // [DR_TB][4]: beta, g, kn . qn
    float* red = sc + DR_TB * 4;                                       // [2][DR_PARTS][DR_COLS][2]
    const int h = blockIdx.x, r = blockIdx.y, c0 = blockIdx.z * DR_COLS;
    const int tid = threadIdx.x, lane = tid & 31, part = tid >> 5;
    const int g = h / (p.heads / p.kv_heads);
    const int t0 = p.q_start[r], n = p.q_start[r + 1] - t0;
    if (n <= 0) return;
    const int col = c0 + lane;
    const bool col_ok = col < dv;
    const int Ck = p.kv_heads * d, W = 2 * Ck + p.heads * dv;
    float* S = p.state + ((size_t)p.slots[r] * p.heads + h) * d * dv;
    float s_reg[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = part + DR_PARTS * i;
        s_reg[i] = (row < d && col_ok) ? S[(size_t)row * dv + col] : 0.f;
    }
    const T* qkv = reinterpret_cast<const T*>(p.qkv);
    const T* proj = reinterpret_cast<const T*>(p.proj);
    const float decay_rate = expf(p.a_log[h]), dtb = p.dt_bias[h];
    const float q_scale = rsqrtf((float)d);
    int buf = 0;
    for (int b0 = 0; b0 < n; b0 += DR_TB) {
        const int nb = min(DR_TB, n - b0);
        __syncthreads();
        // warp w brings token w of the batch: k and q of head g with their norms, this block's columns of v, beta and g
        if (part < nb) {
            const int t = t0 + b0 + part;
            const T* rowp = qkv + (size_t)t * W;
            float sq = 0.f, sk = 0.f;
            for (int e = lane; e < d; e += 32) {
                const float qe = to_f32<T>(rowp[(size_t)g * d + e]), ke = to_f32<T>(rowp[Ck + (size_t)g * d + e]);
                kq[part * d + e] = make_float2(ke, qe);
                sq = fmaf(qe, qe, sq); sk = fmaf(ke, ke, sk);
            }
            sq = warp_sum(sq); sk = warp_sum(sk);
            const float rq = q_scale / sqrtf(sq + 1e-6f), rk = 1.f / sqrtf(sk + 1e-6f);
            float dot = 0.f;
            for (int e = lane; e < d; e += 32) {
                float2 v2 = kq[part * d + e];
                v2.x *= rk; v2.y *= rq;
                kq[part * d + e] = v2;
                dot = fmaf(v2.x, v2.y, dot);
            }
            dot = warp_sum(dot);
            vv[part * DR_COLS + lane] = col_ok ? to_f32<T>(rowp[2 * Ck + (size_t)h * dv + col]) : 0.f;
            if (lane == 0) {
                const float pa = to_f32<T>(proj[(size_t)t * p.proj_stride + p.a_off + h]);
                const float pb = to_f32<T>(proj[(size_t)t * p.proj_stride + p.b_off + h]);
                sc[part * 4] = sigmoidf_(pb);
                sc[part * 4 + 1] = expf(-decay_rate * softplusf_(pa + dtb));
                sc[part * 4 + 2] = dot;
            }
        }
        __syncthreads();
        for (int j = 0; j < nb; ++j) {
            const float2* kqj = kq + j * d;
            float A = 0.f, Q = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                const int row = part + DR_PARTS * i;
                if (row < d) {
                    const float2 v2 = kqj[row];
                    A = fmaf(s_reg[i], v2.x, A);
                    Q = fmaf(s_reg[i], v2.y, Q);
                }
            }
            float* rb = red + buf * (DR_PARTS * DR_COLS * 2);
            rb[(part * DR_COLS + lane) * 2] = A;
            rb[(part * DR_COLS + lane) * 2 + 1] = Q;
            __syncthreads();
            A = 0.f; Q = 0.f;
#pragma unroll
            for (int w = 0; w < DR_PARTS; ++w) {                      // every warp adds the parts in the same order
                A += rb[(w * DR_COLS + lane) * 2];
                Q += rb[(w * DR_COLS + lane) * 2 + 1];
            }
            buf ^= 1;
            const float beta = sc[j * 4], gd = sc[j * 4 + 1], kqd = sc[j * 4 + 2];
            const float u = beta * (vv[j * DR_COLS + lane] - gd * A);
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                const int row = part + DR_PARTS * i;
                if (row < d) s_reg[i] = fmaf(kqj[row].x, u, gd * s_reg[i]);
            }
            if (part == 0 && col_ok) p.out[((size_t)(t0 + b0 + j) * p.heads + h) * dv + col] = fmaf(kqd, u, gd * Q);
        }
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int row = part + DR_PARTS * i;
        if (row < d && col_ok) S[(size_t)row * dv + col] = s_reg[i];
    }
}

MSGL_API int msgl_delta_rule(const void* qkv, const void* proj, long long proj_stride, int a_off, int b_off, const float* a_log,
                             const float* dt_bias, float* state, const int* q_start, const int* slots, float* out, int heads, int kv_heads,
                             int d, int dv, int B, int dtype, cudaStream_t stream) {
    if (B <= 0) return MSGL_OK;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || d <= 0 || dv <= 0 || d > DR_PARTS * 64) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    DeltaParams p;
    p.qkv = qkv; p.proj = proj; p.proj_stride = proj_stride; p.a_off = a_off; p.b_off = b_off; p.a_log = a_log; p.dt_bias = dt_bias;
    p.state = state; p.q_start = q_start; p.slots = slots; p.out = out; p.heads = heads; p.kv_heads = kv_heads; p.d = d; p.dv = dv;
    const dim3 grid(heads, B, (dv + DR_COLS - 1) / DR_COLS);
    const size_t smem = ((size_t)2 * DR_TB * d + DR_TB * DR_COLS + DR_TB * 4 + 2 * DR_PARTS * DR_COLS * 2) * sizeof(float);
    const int rpt = (d + DR_PARTS - 1) / DR_PARTS;
#define DR_LAUNCH(N)                                                                                                        \
    do {                                                                                                                    \
        if (dtype == MSGL_F32) delta_rule_kernel<float, N><<<grid, DR_COLS * DR_PARTS, smem, stream>>>(p);                  \
        else delta_rule_kernel<__nv_bfloat16, N><<<grid, DR_COLS * DR_PARTS, smem, stream>>>(p);                            \
    } while (0)
    if (rpt <= 4) DR_LAUNCH(4);
    else if (rpt <= 8) DR_LAUNCH(8);
    else if (rpt <= 16) DR_LAUNCH(16);
    else if (rpt <= 32) DR_LAUNCH(32);
    else DR_LAUNCH(64);
#undef DR_LAUNCH
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
