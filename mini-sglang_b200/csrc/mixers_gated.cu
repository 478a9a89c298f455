// Kernels of mixers and feed-forwards whose weights over the past are gates rather than a softmax, and of routed experts
// (sm_100a; plain C entry points, loaded by ops.py as the library "mixers_gated", built only for models with such parts):
//
//   embed_positions_kernel     float(E[id]) * c + float(P[position]): opens the float32 stream of a model with learned places
//   headnorm_kvwrite_kernel    per-head RMS norm of q and k (one weight for all heads), q warmed up by its place, K and V rows
//                              (of head sizes of their own) into the paged cache
//   sigmoid_attention_kernel   causal attention whose weight of a key is sigmoid(q.k * scale + bias[head][distance]): no sum
//                              over keys divides anything, so pieces of the keys simply add up (sum_pieces_kernel)
//   sigmoid_attention_mma_kernel   the same for bfloat16 with both products on mma.sync tiles (64 rows a block, float32 scores)
//   mingru_kernel              S_t = (1 - z_t) S_(t-1) + z_t c_t per channel with gates from the current token, times silu(g)
//   mingru_chunk_sum_kernel, mingru_chunk_out_kernel      long portions: chunks of the tokens side by side
//   pair_norm_kernel           c * (rms(a) * wa + rms(b) * wb) in float32: two mixers' outputs joined
//   causal_conv_act_kernel     short causal convolution per channel with bias and silu, continued from a request's last inputs
//                              (causal_conv_act_vec_kernel: 16 bytes of channels a thread where the rows allow it);
//                              conv_state_shift_kernel brings those up to date
//   ssm_scan_kernel            S_t = exp(-exp(A) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t per head, token by token
//   ssm_chunk_state_kernel, ssm_chunk_carry_kernel, ssm_chunk_out_kernel     long portions: chunks of 64 tokens side by side
//                              (a chunk's own sum and decay; the chunks' start states in order; outputs from both)
//   gate_group_norm_kernel     (y * silu(z)) RMS-normed in equal parts of the row, times a weight
//   unary_act_kernel           relu(x)^2 (and the other activations), times a constant
//   route_kernel               router logits in float32, sigmoid scores, correction, limitation to the best groups, the top
//                              experts and their weights: one block per token
//                              (or, in its softmax mode, the largest logits and the softmax over the chosen ones; a further row's
//                              sigmoid per token beside them)
//   expert_gate_up_kernel, expert_down_kernel      the chosen experts' products for a few tokens, straight from the experts'
//                              stacked weights (weight-streaming, one warp per output row); silu(gate) * up or the clamped
//                              form; an extra term (a shared expert's output times a gate per token) joins the sum
//   clamped_glu_kernel         min(gate, limit) * sigmoid(1.702 ...) * (clamp(up) + 1) of a packed [gate | up] row
//   expert_count_kernel, expert_place_kernel, expert_gather_kernel, expert_combine_kernel    many tokens: the (token, choice)
//                              pairs in the order of their experts (stable), rows gathered for one product per expert, and the
//                              weighted sum of every token's rows
//
// Scores, weights, norms, gates, decays, states and everything that enters a recurrence are float32; T is the type of the
// activations between kernels (float or bfloat16).  The order of every sum at a position is fixed by absolute positions, never
// by how the tokens were cut into steps or by what else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float gelu_tanhf_(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
// a gated activation with bounded inputs: g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1)
__device__ __forceinline__ float clamped_gluf_(float gate, float up, float limit) {
    const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
    return g * sigmoidf_(1.702f * g) * (u + 1.f);
}
// ln(1 + e^x) without a threshold: max(x, 0) + ln(1 + e^-|x|)
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// 16 bytes of activations at once: VecOf<T>::N elements to and from float (the address is 16-byte aligned)
template <typename T> struct VecOf;
template <> struct VecOf<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* o) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* o) { *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]); }
};
template <> struct VecOf<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const unsigned u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(u[i] << 16);
            o[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* o) {
        unsigned u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
            u[i] = *reinterpret_cast<const unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(u[0], u[1], u[2], u[3]);
    }
};
__device__ __forceinline__ float act_of(int act, float v) {
    switch (act) {
        case 0: return siluf_(v);
        case 1: return gelu_tanhf_(v);
        case 2: return sigmoidf_(v);
        case 3: return v > 0.f ? v * v : 0.f;
        default: return fmaxf(v, 0.f);
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Embedding with a learned vector per place
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_positions_kernel(const int* __restrict__ ids, const int* __restrict__ positions, const T* __restrict__ table,
                                       const T* __restrict__ places, float* __restrict__ out, int H, int V, int n_places, float c) {
    const int t = blockIdx.x;
    const int id = min(max(ids[t], 0), V - 1), pos = min(max(positions[t], 0), n_places - 1);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[(size_t)t * H + i] = to_f32<T>(table[(size_t)id * H + i]) * c + to_f32<T>(places[(size_t)pos * H + i]);
}

MSGL_API int msgl_embed_positions(const int* ids, const int* positions, const void* table, const void* places, float* out, int T_,
                                  int H, int V, int n_places, float c, int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (H <= 0 || V <= 0 || n_places <= 0) return MSGL_ERR_SIZE;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == MSGL_F32)
        embed_positions_kernel<float><<<T_, threads, 0, stream>>>(ids, positions, (const float*)table, (const float*)places, out, H, V, n_places, c);
    else if (dtype == MSGL_BF16)
        embed_positions_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>(ids, positions, (const __nv_bfloat16*)table,
                                                                          (const __nv_bfloat16*)places, out, H, V, n_places, c);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Per-head RMS norm of q and k, q times a factor that grows with the place, K and V into the paged cache
//
//   proj row: q at q_off (n_q * d), k at k_off (n_kv * d), v at v_off (n_kv * dv)
//   q_out[t, h, :] = q / sqrt(mean(q^2) + eps) * wq * (1 + coef * ln(floor((pos + 1) / every) + 1))
//   K cache [page][kv head][slot][d] <- k / sqrt(mean(k^2) + eps) * wk;  V cache [page][kv head][slot][dv] <- v
// One warp per (token, job), jobs = the q heads, then the k heads, then the v heads.
// ---------------------------------------------------------------------------------------
struct HeadNormParams {
    const void* proj; long long stride; int q_off, k_off, v_off;
    int n_q, n_kv, d, dv;
    const float* wq; const float* wk; float eps;
    float temp_coef; int temp_every;
    const int* positions; const int* out_loc;
    void* q_out; void* k_cache; void* v_cache; int page_size; int T;
};

template <typename T>
__global__ void headnorm_kvwrite_kernel(const HeadNormParams p) {
    const int jobs = p.n_q + 2 * p.n_kv;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= (long long)p.T * jobs) return;
    const int t = (int)(w / jobs), job = (int)(w - (long long)t * jobs);
    const T* row = reinterpret_cast<const T*>(p.proj) + (size_t)t * p.stride;
    if (job < p.n_q) {
        const T* src = row + p.q_off + (size_t)job * p.d;
        float ss = 0.f;
        for (int e = lane; e < p.d; e += 32) { const float v = to_f32<T>(src[e]); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        float f = rsqrtf(ss / (float)p.d + p.eps);
        if (p.temp_coef != 0.f) {
            const int pos = p.positions[t];
            f *= 1.f + p.temp_coef * logf((float)((pos + 1) / p.temp_every) + 1.f);
        }
        T* dst = reinterpret_cast<T*>(p.q_out) + ((size_t)t * p.n_q + job) * p.d;
        for (int e = lane; e < p.d; e += 32) dst[e] = from_f32<T>(to_f32<T>(src[e]) * f * p.wq[e]);
        return;
    }
    if (p.out_loc == nullptr) return;
    const int loc = p.out_loc[t];
    const int page = loc / p.page_size, off = loc - page * p.page_size;
    if (job < p.n_q + p.n_kv) {
        const int g = job - p.n_q;
        const T* src = row + p.k_off + (size_t)g * p.d;
        float ss = 0.f;
        for (int e = lane; e < p.d; e += 32) { const float v = to_f32<T>(src[e]); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float f = rsqrtf(ss / (float)p.d + p.eps);
        T* dst = reinterpret_cast<T*>(p.k_cache) + (((size_t)page * p.n_kv + g) * p.page_size + off) * p.d;
        for (int e = lane; e < p.d; e += 32) dst[e] = from_f32<T>(to_f32<T>(src[e]) * f * p.wk[e]);
    } else {
        const int g = job - p.n_q - p.n_kv;
        const T* src = row + p.v_off + (size_t)g * p.dv;
        T* dst = reinterpret_cast<T*>(p.v_cache) + (((size_t)page * p.n_kv + g) * p.page_size + off) * p.dv;
        for (int e = lane; e < p.dv; e += 32) dst[e] = src[e];
    }
}

MSGL_API int msgl_headnorm_kvwrite(const void* proj, long long stride, int q_off, int k_off, int v_off, int n_q, int n_kv, int d, int dv,
                                   const float* wq, const float* wk, float eps, float temp_coef, int temp_every, const int* positions,
                                   const int* out_loc, void* q_out, void* k_cache, void* v_cache, int page_size, int T_, int dtype,
                                   cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (n_q <= 0 || n_kv <= 0 || d <= 0 || dv <= 0 || page_size < 1 || (temp_coef != 0.f && temp_every < 1)) return MSGL_ERR_SIZE;
    HeadNormParams p;
    p.proj = proj; p.stride = stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.n_q = n_q; p.n_kv = n_kv; p.d = d; p.dv = dv;
    p.wq = wq; p.wk = wk; p.eps = eps; p.temp_coef = temp_coef; p.temp_every = temp_every; p.positions = positions; p.out_loc = out_loc;
    p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache; p.page_size = page_size; p.T = T_;
    const long long warps = (long long)T_ * (n_q + 2 * n_kv);
    const int per_block = 8;
    const unsigned grid = (unsigned)((warps + per_block - 1) / per_block);
    if (dtype == MSGL_F32) headnorm_kvwrite_kernel<float><<<grid, per_block * 32, 0, stream>>>(p);
    else if (dtype == MSGL_BF16) headnorm_kvwrite_kernel<__nv_bfloat16><<<grid, per_block * 32, 0, stream>>>(p);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Causal attention with sigmoid weights over the paged cache
//
//   o[i, h, :] = sum_{j <= i} sigmoid(q[i, h] . k[j, g] * scale + bias[h][min(i - j, L - 1)]) * v[j, g, :]
//
// A block owns a tile of QT tokens x GH query heads of one kv head (SA_ROWS rows, one warp each) and walks the keys in
// chunks of 32 anchored at multiples of 32.  In the score phase lane l of a row's warp takes key l of the chunk, in the value
// phase lane l takes the output elements l, l + 32, ...  With `splits` > 1 (steps in which every request brings one token)
// block z walks the keys [z * split_keys, (z + 1) * split_keys) only and leaves its sums in `part`; the pieces are added in
// order by sum_pieces_kernel.
// ---------------------------------------------------------------------------------------
#define SA_ROWS 8
#define SA_KC 32
#define SA_MAX_DPL 16       // value head sizes up to 512

struct SigmoidAttnParams {
    const void* q;            // [T, n_q, d]
    const void* k_cache; const void* v_cache;
    const int* q_start; const int* kv_len; const int* block_table; int bt_stride;
    int uniform;                                  // every request brings one token: block x takes request x
    const float* bias; int bias_len;              // [n_q][bias_len]
    void* out; long long out_stride;              // [T rows][n_q * dv]
    float* part; int splits, split_keys;          // [splits][T][n_q][dv] float32
    int T, B, n_q, n_kv, d, dv, page_size, QT, GH;
    float scale;
};

template <typename T, int DPL /* output elements per lane: value head sizes up to 32 * DPL */>
__global__ void __launch_bounds__(SA_ROWS * 32) sigmoid_attention_kernel(const SigmoidAttnParams p) {
    extern __shared__ float smem[];
    const int d = p.d, dv = p.dv;
    float* qs = smem;                                // [SA_ROWS][d]
    float* ks = qs + SA_ROWS * d;                    // [SA_KC][d + 1]
    float* vs = ks + SA_KC * (d + 1);                // [SA_KC][dv]
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
    int key_lo = 0, key_hi = p_max + 1;              // keys this block walks: [key_lo, key_hi)
    if (p.splits > 1) {
        key_lo = blockIdx.z * p.split_keys;
        key_hi = min(key_hi, key_lo + p.split_keys);
    }

    const int tl = warp / p.GH, hl = warp - tl * p.GH;
    const int hg = chunk * p.GH + hl;
    const bool row_ok = tl < n_tok && hg < G && tl < p.QT;
    const int head = kvh * G + (row_ok ? hg : 0);
    const int tok = q_base + t0 + (row_ok ? tl : 0);
    const int pos = p_min + tl;
    const T* qg = reinterpret_cast<const T*>(p.q);
    for (int e = lane; e < d; e += 32) qs[warp * d + e] = row_ok ? to_f32<T>(qg[((size_t)tok * p.n_q + head) * d + e]) : 0.f;
    const float* bias = p.bias + (size_t)head * p.bias_len;
    const T* kc = reinterpret_cast<const T*>(p.k_cache);
    const T* vc = reinterpret_cast<const T*>(p.v_cache);
    const int* bt = p.block_table + (size_t)req * p.bt_stride;

    float o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = 0.f;

    for (int key0 = key_lo - key_lo % SA_KC; key0 < key_hi; key0 += SA_KC) {
        __syncthreads();
        for (int idx = tid; idx < SA_KC * d; idx += SA_ROWS * 32) {
            const int kr = idx / d, e = idx - kr * d;
            const int key = key0 + kr;
            float kv = 0.f;
            if (key >= key_lo && key < key_hi) {
                const int page = bt[key / p.page_size];
                kv = to_f32<T>(kc[(((size_t)page * p.n_kv + kvh) * p.page_size + (key % p.page_size)) * d + e]);
            }
            ks[kr * (d + 1) + e] = kv;
        }
        for (int idx = tid; idx < SA_KC * dv; idx += SA_ROWS * 32) {
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
        const bool vis = row_ok && key <= pos && key >= key_lo && key < key_hi;
        float pr = 0.f;
        if (vis) {
            float acc = 0.f;
            const float* qr = qs + warp * d;
            const float* kr = ks + lane * (d + 1);
            for (int e = 0; e < d; ++e) acc = fmaf(qr[e], kr[e], acc);
            pr = sigmoidf_(acc * p.scale + bias[min(pos - key, p.bias_len - 1)]);
        }
        if (__ballot_sync(0xffffffffu, vis) == 0u) continue;        // warp-uniform
        for (int j = 0; j < SA_KC; ++j) {
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
        float* pg = p.part + (((size_t)blockIdx.z * p.T + tok) * p.n_q + head) * dv;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int e = lane + 32 * i;
            if (e < dv) pg[e] = o[i];
        }
        return;
    }
    T* og = reinterpret_cast<T*>(p.out) + (size_t)tok * p.out_stride + (size_t)head * dv;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int e = lane + 32 * i;
        if (e < dv) og[e] = from_f32<T>(o[i]);
    }
}

// ---------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16, prompts and portions): S = Q K^T and O += P V by mma.sync m16n8k16 with
// float32 accumulators, P = sigmoid(S * scale + bias[head][distance]) in float32 between them, rounded to bfloat16 only as
// the operand of the value product.  A block owns 64 rows = 64 / G tokens x the G query heads of one kv head (so a key tile
// serves all its heads) and walks the keys in tiles of 64 anchored at multiples of 64, two tiles in flight (cp.async).
// DK, DV: the head sizes rounded up to a size the kernel is built for; columns beyond d, dv are zero in shared memory.
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
// 1 / (1 + e^-x) with the special-function unit's 2^x and reciprocal (relative error about 2^-21; -inf gives 0)
__device__ __forceinline__ float fast_sigmoid(float x) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(-1.4426950408889634f * x));
    return __fdividef(1.f, 1.f + e);
}
}  // namespace

#define SAM_R 64            // rows of a block
#define SAM_KT 64           // keys of a tile
#define SAM_THREADS 128
#define SAM_BS_HEADS 8      // heads of a block whose bias entries go through shared memory
#define SAM_BS_LD 136

template <int DK, int DV>
__global__ void __launch_bounds__(SAM_THREADS) sigmoid_attention_mma_kernel(const SigmoidAttnParams p) {
    constexpr int LDK = DK + 8, LDV = DV + 8;           // padded rows (elements): ldmatrix without bank conflicts
    constexpr int NKB = SAM_KT / 8, NDB = DV / 8;
    constexpr int CHK = DK / 8, CHV = DV / 8;           // 16-byte pieces of a row
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [64][LDK]
    __nv_bfloat16* KVs = Qs + SAM_R * LDK;                                          // [stage][K: 64 x LDK | V: 64 x LDV]
    __shared__ float bias_s[SAM_BS_HEADS * SAM_BS_LD];
    __shared__ int tile_sh[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.n_q / p.n_kv;
    const int Gc = G <= SAM_R ? G : SAM_R;
    const int n_chunks = G <= SAM_R ? 1 : (G + SAM_R - 1) / SAM_R;
    const int QT = G <= SAM_R ? SAM_R / G : 1;
    const int kvh = blockIdx.y / n_chunks, chunk = blockIdx.y - kvh * n_chunks;
    if (tid == 0) {
        if (p.uniform) {
            tile_sh[0] = blockIdx.x; tile_sh[1] = 0;
        } else {
            // heaviest tiles first: the last tiles of a request walk the most keys, and blocks start in index order
            int left = (int)gridDim.x - 1 - (int)blockIdx.x, found = -1, at = 0;
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
    // key tiles this block walks: all up to the last position's, or (one-token steps) those of its piece; a piece is a whole
    // number of tiles, so a tile never holds keys of two pieces
    int kt_lo = 0, kt_hi = p_max / SAM_KT + 1;
    if (p.splits > 1) {
        kt_lo = (int)blockIdx.z * (p.split_keys / SAM_KT);
        kt_hi = min(kt_hi, kt_lo + p.split_keys / SAM_KT);
        if (kt_lo >= kt_hi) return;
    }
    const int d = p.d, dv = p.dv;
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(p.k_cache);
    const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(p.v_cache);
    const int* bt = p.block_table + (size_t)req * p.bt_stride;
    const unsigned q_s = smem_u32(Qs), kv_s = smem_u32(KVs);
    constexpr unsigned K_BYTES = SAM_KT * LDK * 2u, STAGE_BYTES = K_BYTES + SAM_KT * LDV * 2u;

    // ---- the block's query rows (zero where the tile has no token or head, and beyond d)
    for (int idx = tid; idx < SAM_R * CHK; idx += SAM_THREADS) {
        const int r = idx / CHK, c = idx - r * CHK;
        const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * SAM_R + hl;
        const bool valid = tl < n_tok && tl < QT && hg < G && c * 8 < d;
        const size_t tok = (size_t)(q_base + t0 + (valid ? tl : 0));
        const __nv_bfloat16* src = qg + (tok * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * d + (valid ? c * 8 : 0);
        cp_async16_u32(q_s + (unsigned)(r * LDK + c * 8) * 2u, src, valid);
    }
    // a thread copies half a row of K and of V per tile: row tid / 2, every second 16-byte piece
    const int ld_row = tid >> 1, ld_half = tid & 1;
    auto load_kv = [&](int stage, int kt) {
        const int key = kt * SAM_KT + ld_row;
        const bool live = key <= p_max;
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

    const int row_base = warp * 16;
    const bool warp_live = row_base / Gc < n_tok;       // else all 16 rows of the warp are empty: it copies, but multiplies nothing
    const int r_lo = row_base + (lane >> 2), r_hi = r_lo + 8;
    const int tl_lo = r_lo / Gc, tl_hi = r_hi / Gc;
    const int hl_lo = r_lo - tl_lo * Gc, hl_hi = r_hi - tl_hi * Gc;
    const int pos_lo = p_min + tl_lo, pos_hi = p_min + tl_hi;
    const float* bias_lo = p.bias + (size_t)min(kvh * G + chunk * SAM_R + hl_lo, p.n_q - 1) * p.bias_len;
    const float* bias_hi = p.bias + (size_t)min(kvh * G + chunk * SAM_R + hl_hi, p.n_q - 1) * p.bias_len;
    // The bias of a key tile through shared memory: entry j of a head stands for the distance dmin + j with dmin = p_min - (last
    // key of the tile), and the row of token tl reads key kk of the tile at tl + 63 - kk.
    const bool bias_staged = Gc <= SAM_BS_HEADS;
    const float* bs_lo = bias_s + hl_lo * SAM_BS_LD + tl_lo + (SAM_KT - 1) - (lane & 3) * 2;
    const float* bs_hi = bias_s + hl_hi * SAM_BS_LD + tl_hi + (SAM_KT - 1) - (lane & 3) * 2;
    const unsigned q_a = q_s + (unsigned)((row_base + (lane & 15)) * LDK + (lane >> 4) * 8) * 2u;
    const unsigned k_lane = (unsigned)(((lane & 7) + ((lane >> 4) & 1) * 8) * LDK + ((lane >> 3) & 1) * 8) * 2u;
    const unsigned v_lane = (unsigned)(((lane & 7) + ((lane >> 3) & 1) * 8) * LDV + ((lane >> 4) & 1) * 8) * 2u;

    float o[NDB][4];
#pragma unroll
    for (int i = 0; i < NDB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    for (int kt = kt_lo; kt < kt_hi; ++kt) {
        const int stage = (kt - kt_lo) & 1;
        if (bias_staged) {       // written before the barrier below, read after it, and not written again before the one that ends the tile
            const int dmin = p_min - (kt * SAM_KT + SAM_KT - 1), span = QT + SAM_KT - 1;
            for (int idx = tid; idx < Gc * span; idx += SAM_THREADS) {
                const int hl = idx / span, j = idx - hl * span;
                const int head = min(kvh * G + chunk * SAM_R + hl, p.n_q - 1);
                bias_s[hl * SAM_BS_LD + j] = p.bias[(size_t)head * p.bias_len + min(max(dmin + j, 0), p.bias_len - 1)];
            }
        }
        if (kt + 1 < kt_hi) {
            load_kv(stage ^ 1, kt + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key0 = kt * SAM_KT;
        if (!warp_live || key0 > p_min + (row_base + 15) / Gc) {      // no row of the warp sees a key of this tile
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
        // ---- weights: every key by itself
        const bool need_mask = key0 + SAM_KT - 1 > p_min;
#pragma unroll
        for (int nb = 0; nb < NKB; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                const int pos = (e < 2) ? pos_lo : pos_hi;
                float w = 0.f;
                if (!need_mask || key <= pos) {
                    const float b = bias_staged ? ((e < 2) ? bs_lo : bs_hi)[-(nb * 8 + (e & 1))]
                                                : ((e < 2) ? bias_lo : bias_hi)[min(max(pos - key, 0), p.bias_len - 1)];
                    w = fast_sigmoid(fmaf(s[nb][e], p.scale, b));
                }
                s[nb][e] = w;
            }
        }
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

    __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(p.out);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int tl = half ? tl_hi : tl_lo, hl = half ? hl_hi : hl_lo, hg = chunk * SAM_R + hl;
        if (!(tl < n_tok && tl < QT && hg < G)) continue;
        if (p.splits > 1) {
            float* pg = p.part + (((size_t)blockIdx.z * p.T + (q_base + t0 + tl)) * p.n_q + (kvh * G + hg)) * dv;
#pragma unroll
            for (int nd = 0; nd < NDB; ++nd) {
                const int col = nd * 8 + (lane & 3) * 2;
                if (col < dv) *reinterpret_cast<float2*>(pg + col) = make_float2(o[nd][half * 2], o[nd][half * 2 + 1]);
            }
            continue;
        }
        __nv_bfloat16* dst = og + (size_t)(q_base + t0 + tl) * p.out_stride + (size_t)(kvh * G + hg) * dv;
#pragma unroll
        for (int nd = 0; nd < NDB; ++nd) {
            const int col = nd * 8 + (lane & 3) * 2;
            if (col < dv)           // dv is a multiple of 8: a pair lies inside the row or outside it
                *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[nd][half * 2], o[nd][half * 2 + 1]);
        }
    }
}

// out[t, c] = sum over the pieces s, in order, of part[s][t][c]; only the pieces that hold keys of the token's request
template <typename T>
__global__ void sum_pieces_kernel(const float* __restrict__ part, const int* __restrict__ kv_len, const int* __restrict__ token_req,
                                  T* __restrict__ out, long long out_stride, int T_, int N, int splits, int split_keys) {
    const int t = blockIdx.x;
    const int r = token_req ? token_req[t] : t;
    const int used = min(splits, (kv_len[r] + split_keys - 1) / split_keys);
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < N; c += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < used; ++s) acc += part[((size_t)s * T_ + t) * N + c];
        out[(size_t)t * out_stride + c] = from_f32<T>(acc);
    }
}

MSGL_API int msgl_sigmoid_attention(const void* q, const void* k_cache, const void* v_cache, const int* q_start, const int* kv_len,
                                    const int* block_table, int bt_stride, int uniform, int n_tiles, const float* bias, int bias_len,
                                    void* out, long long out_stride, float* part, int splits, int split_keys, int T_, int B, int n_q,
                                    int n_kv, int d, int dv, int page_size, int QT, int GH, float scale, int dtype, cudaStream_t stream) {
    if (n_tiles <= 0) return MSGL_OK;
    if (d <= 0 || dv <= 0 || dv > 32 * SA_MAX_DPL || d > 32 * SA_MAX_DPL || n_kv <= 0 || n_q % n_kv || QT < 1 || GH < 1 ||
        QT * GH > SA_ROWS || page_size < 1 || bias == nullptr || bias_len < 1 || splits < 1 ||
        (splits > 1 && (!uniform || part == nullptr || split_keys < SA_KC || split_keys % SA_KC)))
        return MSGL_ERR_SIZE;
    SigmoidAttnParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
    p.bt_stride = bt_stride; p.uniform = uniform; p.bias = bias; p.bias_len = bias_len; p.out = out; p.out_stride = out_stride;
    p.part = part; p.splits = splits; p.split_keys = split_keys; p.T = T_; p.B = B; p.n_q = n_q; p.n_kv = n_kv; p.d = d; p.dv = dv;
    p.page_size = page_size; p.QT = QT; p.GH = GH; p.scale = scale;
    const int G = n_q / n_kv;
    const dim3 grid(n_tiles, n_kv * ((G + GH - 1) / GH), splits);
    const size_t smem = ((size_t)SA_ROWS * d + (size_t)SA_KC * (d + 1) + (size_t)SA_KC * dv) * sizeof(float);
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const int dpl = (dv + 31) / 32;
#define SA_LAUNCH(N)                                                                                                         \
    do {                                                                                                                     \
        static MsglOncePerDevice once;                                                                                       \
        if (smem > 48 * 1024 && once.due()) {                                                                                \
            cudaFuncSetAttribute(sigmoid_attention_kernel<float, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            cudaFuncSetAttribute(sigmoid_attention_kernel<__nv_bfloat16, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            once.mark();                                                                                                     \
        }                                                                                                                    \
        if (dtype == MSGL_F32) sigmoid_attention_kernel<float, N><<<grid, SA_ROWS * 32, smem, stream>>>(p);                  \
        else sigmoid_attention_kernel<__nv_bfloat16, N><<<grid, SA_ROWS * 32, smem, stream>>>(p);                            \
    } while (0)
    if (dpl <= 1) SA_LAUNCH(1);
    else if (dpl <= 2) SA_LAUNCH(2);
    else if (dpl <= 3) SA_LAUNCH(3);
    else if (dpl <= 4) SA_LAUNCH(4);
    else if (dpl <= 8) SA_LAUNCH(8);
    else SA_LAUNCH(16);
#undef SA_LAUNCH
    int code = msgl_check_launch();
    if (code != MSGL_OK || splits <= 1) return code;
    const int N = n_q * dv;
    const dim3 g2(T_, max(1, min((N + 255) / 256, 16)));
    if (dtype == MSGL_F32) sum_pieces_kernel<float><<<g2, 256, 0, stream>>>(part, kv_len, nullptr, (float*)out, out_stride, T_, N, splits, split_keys);
    else sum_pieces_kernel<__nv_bfloat16><<<g2, 256, 0, stream>>>(part, kv_len, nullptr, (__nv_bfloat16*)out, out_stride, T_, N, splits, split_keys);
    return msgl_check_launch();
}

// The tensor-core launch: bfloat16, head sizes that are multiples of 8 up to 128, rows of `out` that pairs of elements can be
// stored into.  n_tiles: the sum over the requests of ceil(tokens / QT) with QT = 64 / (heads per kv head) (1 beyond 64), or
// with `uniform` (every request brings one token) the number of requests; then `splits` pieces of `split_keys` keys (a
// multiple of 64) go to blocks of their own, which leave float32 sums in `part` for sum_pieces_kernel.
MSGL_API int msgl_sigmoid_attention_mma(const void* q, const void* k_cache, const void* v_cache, const int* q_start, const int* kv_len,
                                        const int* block_table, int bt_stride, int uniform, int n_tiles, const float* bias, int bias_len,
                                        void* out, long long out_stride, float* part, int splits, int split_keys, int T_, int B, int n_q,
                                        int n_kv, int d, int dv, int page_size, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return MSGL_OK;
    if (d <= 0 || dv <= 0 || d > 128 || dv > 128 || d % 8 || dv % 8 || n_kv <= 0 || n_q % n_kv || page_size < 1 || bias == nullptr ||
        bias_len < 1 || (out_stride & 1) || ((size_t)out & 3) || splits < 1 ||
        (splits > 1 && (!uniform || part == nullptr || split_keys < SAM_KT || split_keys % SAM_KT || ((size_t)part & 7))))
        return MSGL_ERR_SIZE;
    SigmoidAttnParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
    p.bt_stride = bt_stride; p.uniform = uniform; p.bias = bias; p.bias_len = bias_len; p.out = out; p.out_stride = out_stride;
    p.part = part; p.splits = splits; p.split_keys = split_keys; p.T = T_; p.B = B; p.n_q = n_q; p.n_kv = n_kv; p.d = d; p.dv = dv;
    p.page_size = page_size; p.QT = 0; p.GH = 0; p.scale = scale;
    const int G = n_q / n_kv;
    const dim3 grid(n_tiles, n_kv * (G <= SAM_R ? 1 : (G + SAM_R - 1) / SAM_R), splits);
#define SAM_LAUNCH(DK, DV)                                                                                                   \
    do {                                                                                                                     \
        const size_t smem = ((size_t)SAM_R * (DK + 8) + 2 * ((size_t)SAM_KT * (DK + 8) + (size_t)SAM_KT * (DV + 8))) * 2;    \
        static MsglOncePerDevice once;                                                                                       \
        if (once.due()) {                                                                                                    \
            cudaFuncSetAttribute(sigmoid_attention_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            once.mark();                                                                                                     \
        }                                                                                                                    \
        sigmoid_attention_mma_kernel<DK, DV><<<grid, SAM_THREADS, smem, stream>>>(p);                                        \
    } while (0)
#define SAM_BY_DV(DK)                                                                                                        \
    do {                                                                                                                     \
        if (dv <= 64) SAM_LAUNCH(DK, 64);                                                                                    \
        else if (dv <= 96) SAM_LAUNCH(DK, 96);                                                                               \
        else SAM_LAUNCH(DK, 128);                                                                                            \
    } while (0)
    if (d <= 64) SAM_BY_DV(64);
    else if (d <= 96) SAM_BY_DV(96);
    else SAM_BY_DV(128);
#undef SAM_BY_DV
#undef SAM_LAUNCH
    int code = msgl_check_launch();
    if (code != MSGL_OK || splits <= 1) return code;
    const int N = n_q * dv;
    const dim3 g2(T_, max(1, min((N + 255) / 256, 16)));
    sum_pieces_kernel<__nv_bfloat16><<<g2, 256, 0, stream>>>(part, kv_len, nullptr, (__nv_bfloat16*)out, out_stride, T_, N, splits, split_keys);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// minGRU: a gated recurrence per channel whose gates read the current token only
//
//   z = sigmoid(pz + bz), a = px + bx, c = a + 1/2 (a >= 0) or sigmoid(a) (a < 0)
//   S_t = (1 - z_t) S_(t-1) + z_t c_t;   out_t = S_t * silu(pg_t) * c_out
//   pz, px, pg: columns of one packed projection; state [slot][W] float32
// One thread per (request, channel) walks the request's tokens of the step in order.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void mingru_kernel(const void* proj_, long long stride, int z_off, int x_off, int g_off, int W,
                              const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
                              const int* __restrict__ q_start, const int* __restrict__ slots, void* out_, long long out_stride,
                              float c_out) {
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int t0 = q_start[r], n = q_start[r + 1] - t0;
    if (n <= 0) return;
    const T* proj = reinterpret_cast<const T*>(proj_);
    T* out = reinterpret_cast<T*>(out_);
    float* Sp = state + (size_t)slots[r] * W + c;
    float S = *Sp;
    const float b_z = bz[c], b_x = bx[c];
    const T* row = proj + (size_t)t0 * stride;
    float pz = to_f32<T>(row[z_off + c]), px = to_f32<T>(row[x_off + c]), pg = to_f32<T>(row[g_off + c]);
    for (int tt = 0; tt < n; ++tt) {
        float nz = 0.f, nx = 0.f, ng = 0.f;
        if (tt + 1 < n) {                              // the next token's numbers are on their way while this one is computed
            const T* nrow = proj + (size_t)(t0 + tt + 1) * stride;
            nz = to_f32<T>(nrow[z_off + c]); nx = to_f32<T>(nrow[x_off + c]); ng = to_f32<T>(nrow[g_off + c]);
        }
        const float z = sigmoidf_(pz + b_z), a = px + b_x;
        const float cand = a >= 0.f ? a + 0.5f : sigmoidf_(a);
        S = (1.f - z) * S + z * cand;
        out[(size_t)(t0 + tt) * out_stride + c] = from_f32<T>(S * siluf_(pg) * c_out);
        pz = nz; px = nx; pg = ng;
    }
    *Sp = S;
}

MSGL_API int msgl_mingru(const void* proj, long long stride, int z_off, int x_off, int g_off, int W, const float* bz, const float* bx,
                         float* state, const int* q_start, const int* slots, void* out, long long out_stride, float c_out, int B,
                         int dtype, cudaStream_t stream) {
    if (B <= 0) return MSGL_OK;
    if (W <= 0) return MSGL_ERR_SIZE;
    const int threads = 64;
    const dim3 grid((W + threads - 1) / threads, B);
    if (dtype == MSGL_F32) mingru_kernel<float><<<grid, threads, 0, stream>>>(proj, stride, z_off, x_off, g_off, W, bz, bx, state, q_start, slots, out, out_stride, c_out);
    else if (dtype == MSGL_BF16) mingru_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(proj, stride, z_off, x_off, g_off, W, bz, bx, state, q_start, slots, out, out_stride, c_out);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// minGRU over long portions: the tokens of a request in chunks of `L` that run side by side.  The recurrence S_t = a_t S_(t-1) + b_t
// (a = 1 - z, b = z * candidate) of a chunk is S_end = A S_start + E with A = the product of its a and E = its end state from
// zero.  mingru_chunk_sum_kernel leaves (A, E) of every chunk in `sums` [chunk][2][W] and the request's state before the step in
// `init` [request][W]; mingru_chunk_out_kernel brings a chunk's S_start up from `init` through the chunks before it, walks
// the chunk and writes the outputs; the last chunk of a request writes the state back.  Float32 throughout; the result differs
// from the token-by-token kernel by rounding only.  Block y = chunk (over all requests, in order), thread = channel.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ bool find_chunk_y(const int* __restrict__ q_start, int B, int L, int* sh, int& req, int& first, int& c0) {
    if (threadIdx.x == 0) {
        int left = blockIdx.y, found = -1, base = 0;
        for (int r = 0; r < B; ++r) {
            const int nc = (q_start[r + 1] - q_start[r] + L - 1) / L;
            if (left < nc) { found = r; break; }
            left -= nc; base += nc;
        }
        sh[0] = found; sh[1] = base; sh[2] = left;
    }
    __syncthreads();
    req = sh[0]; first = sh[1]; c0 = sh[2];
    return req >= 0;
}

template <typename T>
__global__ void mingru_chunk_sum_kernel(const void* proj_, long long stride, int z_off, int x_off, int W, const float* __restrict__ bz,
                                        const float* __restrict__ bx, const float* __restrict__ state, const int* __restrict__ q_start,
                                        const int* __restrict__ slots, int B, int L, float* __restrict__ sums, float* __restrict__ init) {
    __shared__ int sh[3];
    int r, first, ci;
    if (!find_chunk_y(q_start, B, L, sh, r, first, ci)) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    if (ci == 0) init[(size_t)r * W + c] = state[(size_t)slots[r] * W + c];
    const int t0 = q_start[r] + ci * L, n = min(L, q_start[r + 1] - t0);
    const T* proj = reinterpret_cast<const T*>(proj_);
    const float b_z = bz[c], b_x = bx[c];
    float A = 1.f, E = 0.f;
    for (int tt = 0; tt < n; ++tt) {
        const T* row = proj + (size_t)(t0 + tt) * stride;
        const float z = sigmoidf_(to_f32<T>(row[z_off + c]) + b_z), a = to_f32<T>(row[x_off + c]) + b_x;
        const float cand = a >= 0.f ? a + 0.5f : sigmoidf_(a);
        A *= 1.f - z;
        E = (1.f - z) * E + z * cand;
    }
    float* o = sums + (size_t)(first + ci) * 2 * W;
    o[c] = A; o[W + c] = E;
}

template <typename T>
__global__ void mingru_chunk_out_kernel(const void* proj_, long long stride, int z_off, int x_off, int g_off, int W,
                                        const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
                                        const int* __restrict__ q_start, const int* __restrict__ slots, int B, int L,
                                        const float* __restrict__ sums, const float* __restrict__ init, void* out_, long long out_stride,
                                        float c_out) {
    __shared__ int sh[3];
    int r, first, ci;
    if (!find_chunk_y(q_start, B, L, sh, r, first, ci)) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    float S = init[(size_t)r * W + c];
    for (int k = 0; k < ci; ++k) {
        const float* o = sums + (size_t)(first + k) * 2 * W;
        S = fmaf(o[c], S, o[W + c]);
    }
    const int t0 = q_start[r] + ci * L, n = min(L, q_start[r + 1] - t0);
    const T* proj = reinterpret_cast<const T*>(proj_);
    T* out = reinterpret_cast<T*>(out_);
    const float b_z = bz[c], b_x = bx[c];
    for (int tt = 0; tt < n; ++tt) {
        const T* row = proj + (size_t)(t0 + tt) * stride;
        const float z = sigmoidf_(to_f32<T>(row[z_off + c]) + b_z), a = to_f32<T>(row[x_off + c]) + b_x;
        const float pg = to_f32<T>(row[g_off + c]);
        const float cand = a >= 0.f ? a + 0.5f : sigmoidf_(a);
        S = (1.f - z) * S + z * cand;
        out[(size_t)(t0 + tt) * out_stride + c] = from_f32<T>(S * siluf_(pg) * c_out);
    }
    if (t0 + n == q_start[r + 1]) state[(size_t)slots[r] * W + c] = S;
}

// n_chunks: the sum over the requests of ceil(tokens / L); sums: float32 [n_chunks][2][W]; init: float32 [B][W]
MSGL_API int msgl_mingru_chunked(const void* proj, long long stride, int z_off, int x_off, int g_off, int W, const float* bz, const float* bx,
                                 float* state, const int* q_start, const int* slots, void* out, long long out_stride, float c_out, int B,
                                 int L, int n_chunks, float* sums, float* init, int dtype, cudaStream_t stream) {
    if (B <= 0 || n_chunks <= 0) return MSGL_OK;
    if (W <= 0 || L < 1 || sums == nullptr || init == nullptr || n_chunks > 65535) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const int threads = 128;
    const dim3 grid((W + threads - 1) / threads, n_chunks);
    if (dtype == MSGL_F32) {
        mingru_chunk_sum_kernel<float><<<grid, threads, 0, stream>>>(proj, stride, z_off, x_off, W, bz, bx, state, q_start, slots, B, L, sums, init);
        mingru_chunk_out_kernel<float><<<grid, threads, 0, stream>>>(proj, stride, z_off, x_off, g_off, W, bz, bx, state, q_start, slots, B, L, sums, init, out, out_stride, c_out);
    } else {
        mingru_chunk_sum_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(proj, stride, z_off, x_off, W, bz, bx, state, q_start, slots, B, L, sums, init);
        mingru_chunk_out_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(proj, stride, z_off, x_off, g_off, W, bz, bx, state, q_start, slots, B, L, sums, init, out, out_stride, c_out);
    }
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// out = c * (a / rms(a) * wa + b / rms(b) * wb) in float32: the outputs of two mixers joined, each normed over the row
// One block per token.
// ---------------------------------------------------------------------------------------
template <typename A>
__global__ void __launch_bounds__(256) pair_norm_kernel(const A* __restrict__ a, const A* __restrict__ b, const float* __restrict__ wa,
                                                        const float* __restrict__ wb, float eps, float c, float* __restrict__ out, int H) {
    __shared__ float scratch[32];
    const size_t t = blockIdx.x;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float x = to_f32<A>(a[t * H + i]), y = to_f32<A>(b[t * H + i]);
        sa = fmaf(x, x, sa); sb = fmaf(y, y, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float fa = rsqrtf(sa / (float)H + eps) * c, fb = rsqrtf(sb / (float)H + eps) * c;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[t * H + i] = to_f32<A>(a[t * H + i]) * fa * wa[i] + to_f32<A>(b[t * H + i]) * fb * wb[i];
}

MSGL_API int msgl_pair_norm(const void* a, const void* b, int in_is_f32, const float* wa, const float* wb, float eps, float c, float* out,
                            int T_, int H, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (H <= 0) return MSGL_ERR_SIZE;
    if (in_is_f32) pair_norm_kernel<float><<<T_, 256, 0, stream>>>((const float*)a, (const float*)b, wa, wb, eps, c, out, H);
    else pair_norm_kernel<__nv_bfloat16><<<T_, 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, wa, wb, eps, c, out, H);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Short causal convolution per channel with bias and an activation, continued from the request's last inputs
//
//   y[t, c] = act(bias[c] + sum_j w[j][c] * u[t - (K - 1) + j, c]);  w comes transposed, [K][C], the oldest input's tap first;
//   inputs before the step's first token come from state [slot][K - 1][C] (oldest first; zero when the request was opened)
// One thread per (token, channel).  conv_state_shift_kernel then moves the request's last K - 1 inputs into the state.
// ---------------------------------------------------------------------------------------
#define CV_MAX_TAPS 16
template <typename T>
__global__ void causal_conv_act_kernel(const void* in_, long long stride, int off, int C, int K, const float* __restrict__ w,
                                       const float* __restrict__ bias, const void* state_, const int* __restrict__ token_req,
                                       const int* __restrict__ q_start, const int* __restrict__ slots, void* out_, int act) {
    const int t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const T* in = reinterpret_cast<const T*>(in_);
    const T* state = reinterpret_cast<const T*>(state_);
    const int r = token_req[t];
    const int local = t - q_start[r];
    const int slot = slots[r];
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < K; ++j) {
        const int li = local - (K - 1) + j;              // place of the input among the step's tokens of the request
        float u;
        if (li >= 0) u = to_f32<T>(in[(size_t)(t - (K - 1) + j) * stride + off + c]);
        else u = to_f32<T>(state[((size_t)slot * (K - 1) + (K - 1 + li)) * C + c]);
        acc = fmaf(w[(size_t)j * C + c], u, acc);
    }
    if (act == 0) acc = siluf_(acc);
    reinterpret_cast<T*>(out_)[(size_t)t * C + c] = from_f32<T>(acc);
}

// The same with 16 bytes of channels a thread and `tb` tokens in turn (CV_TB in a long step, 1 in a short one, where the tokens
// are better walked side by side), for up to 4 taps: the request's last three inputs stay in registers from token to token.  A tap that does not exist (fewer than 4) has weight 0 and is not read; the sum of a token is the
// same sequence of multiply-adds as above.
#define CV_TB 8
template <typename T>
__global__ void __launch_bounds__(128)
causal_conv_act_vec_kernel(const void* in_, long long stride, int off, int C, int K, const float* __restrict__ w, const float* __restrict__ bias,
                           const void* state_, const int* __restrict__ token_req, const int* __restrict__ q_start,
                           const int* __restrict__ slots, void* out_, int act, int T_, int tb) {
    constexpr int V = VecOf<T>::N;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (c >= C) return;
    const T* in = reinterpret_cast<const T*>(in_) + off + c;
    const T* state = reinterpret_cast<const T*>(state_);
    T* out = reinterpret_cast<T*>(out_) + c;
    const int skip = 4 - K;
    float wv[4][V], bv[V], win[3][V];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < V; ++i) wv[j][i] = j >= skip ? w[(size_t)(j - skip) * C + c + i] : 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) bv[i] = bias ? bias[c + i] : 0.f;
    int prev = -1;
    for (int tt = 0; tt < tb; ++tt) {
        const int t = blockIdx.y * tb + tt;
        if (t >= T_) break;
        const int r = token_req[t];
        if (r != prev) {                                 // the window of the request's inputs before t
            const int local = t - q_start[r], slot = slots[r];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int li = local - 3 + j;
                if (j >= skip) {
                    if (li >= 0) VecOf<T>::load(in + (size_t)(t - 3 + j) * stride, win[j]);
                    else VecOf<T>::load(state + ((size_t)slot * (K - 1) + (K - 1 + li)) * C + c, win[j]);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) win[j][i] = 0.f;
                }
            }
            prev = r;
        }
        float cur[V], o[V];
        VecOf<T>::load(in + (size_t)t * stride, cur);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float acc = bv[i];
            acc = fmaf(wv[0][i], win[0][i], acc);
            acc = fmaf(wv[1][i], win[1][i], acc);
            acc = fmaf(wv[2][i], win[2][i], acc);
            acc = fmaf(wv[3][i], cur[i], acc);
            o[i] = act == 0 ? siluf_(acc) : acc;
            win[0][i] = win[1][i]; win[1][i] = win[2][i]; win[2][i] = cur[i];
        }
        VecOf<T>::store(out + (size_t)t * C, o);
    }
}

template <typename T>
__global__ void conv_state_shift_kernel(const void* in_, long long stride, int off, int C, int K, void* state_,
                                        const int* __restrict__ q_start, const int* __restrict__ slots) {
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const T* in = reinterpret_cast<const T*>(in_);
    T* state = reinterpret_cast<T*>(state_) + (size_t)slots[r] * (K - 1) * C;
    const int t0 = q_start[r], n = q_start[r + 1] - t0;
    if (n <= 0) return;
    for (int i = 0; i < K - 1; ++i) {                    // row i of the new state is row i + n of [old state; the step's inputs]
        const int s = i + n;
        state[(size_t)i * C + c] = s < K - 1 ? state[(size_t)s * C + c] : in[(size_t)(t0 + s - (K - 1)) * stride + off + c];
    }
}

MSGL_API int msgl_causal_conv_act(const void* in, long long stride, int off, int C, int K, const float* w, const float* bias, void* state,
                                  const int* token_req, const int* q_start, const int* slots, void* out, int act, int T_, int B,
                                  int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (C <= 0 || K < 1 || K > CV_MAX_TAPS || (K > 1 && state == nullptr)) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const int threads = 128;
    const int V = dtype == MSGL_F32 ? 4 : 8;
    const size_t item = dtype == MSGL_F32 ? 4 : 2;
    const bool vec = K <= 4 && C % V == 0 && stride % V == 0 && off % V == 0 && ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
                     ((uintptr_t)state % 16) == 0 && (stride * (long long)item) % 16 == 0;
    if (vec) {
        const int tb = T_ >= 64 * CV_TB ? CV_TB : 1;
        const dim3 grid((C / V + threads - 1) / threads, (T_ + tb - 1) / tb);
        if (dtype == MSGL_F32) causal_conv_act_vec_kernel<float><<<grid, threads, 0, stream>>>(in, stride, off, C, K, w, bias, state, token_req, q_start, slots, out, act, T_, tb);
        else causal_conv_act_vec_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(in, stride, off, C, K, w, bias, state, token_req, q_start, slots, out, act, T_, tb);
    } else {
        const dim3 grid((C + threads - 1) / threads, T_);
        if (dtype == MSGL_F32) causal_conv_act_kernel<float><<<grid, threads, 0, stream>>>(in, stride, off, C, K, w, bias, state, token_req, q_start, slots, out, act);
        else causal_conv_act_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(in, stride, off, C, K, w, bias, state, token_req, q_start, slots, out, act);
    }
    int code = msgl_check_launch();
    if (code != MSGL_OK || K == 1) return code;
    const dim3 g2((C + threads - 1) / threads, B);
    if (dtype == MSGL_F32) conv_state_shift_kernel<float><<<g2, threads, 0, stream>>>(in, stride, off, C, K, state, q_start, slots);
    else conv_state_shift_kernel<__nv_bfloat16><<<g2, threads, 0, stream>>>(in, stride, off, C, K, state, q_start, slots);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// State-space scan, token by token
//
//   per head h (group g = h / (heads / groups)), state S [N][P] float32 per request:
//     dt = softplus(pdt[t, h] + dt_bias[h]);  S <- exp(-exp(A_log[h]) * dt) * S + dt * B[t, g, :] x[t, h, :]^T
//     y[t, h, :] = S^T C[t, g, :] + D[h] * x[t, h, :]
//   xbc row [T][heads * P | groups * N | groups * N] (what the convolution left); pdt a column range of the packed projection
// A block owns SS_COLS columns of one (request, head) state and walks the request's tokens in order; SS_PARTS threads share
// a column's rows.
// ---------------------------------------------------------------------------------------
#define SS_COLS 32
#define SS_PARTS 8
#define SS_MAX_ROWS 64      // state sizes up to SS_PARTS * SS_MAX_ROWS
#define SS_TB 8             // tokens whose B, C, x, decay and step lie in shared memory together

// The tokens go through shared memory in batches of SS_TB, two batches in flight: a thread loads its share of the next batch into
// registers before it walks the current one and puts them down afterwards, so a token costs its multiply-adds, not a wait for
// memory.  A batch row is [B: N | C: N | x: SS_COLS | decay | step]; the thread that brings a token's dt makes decay and step.
// The sums of a token are the same, in the same order, however the tokens were cut into steps.
template <typename T, int NR>
__global__ void __launch_bounds__(SS_COLS * SS_PARTS)
ssm_scan_kernel(const void* xbc_, int heads, int groups, int N, int P, const void* proj_, long long stride, int dt_off,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
                float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ slots, float* __restrict__ y) {
    extern __shared__ float sm[];                    // [2][SS_TB][2 N + SS_COLS + 2]
    constexpr int NT = SS_COLS * SS_PARTS;
    constexpr int PF = (SS_TB * (2 * SS_PARTS * NR + SS_COLS + 1) + NT - 1) / NT;
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * SS_COLS;
    const int tid = threadIdx.x;
    const int part = tid & (SS_PARTS - 1), col = col0 + (tid >> 3);
    const bool col_ok = col < P;
    const int t0 = q_start[r], n = q_start[r + 1] - t0;
    if (n <= 0) return;
    const int g = h / (heads / groups);
    const int inner = heads * P, C_ = inner + 2 * groups * N;
    const T* xbc = reinterpret_cast<const T*>(xbc_);
    const T* proj = reinterpret_cast<const T*>(proj_);
    float* S = state + (((size_t)slots[r] * heads + h) * N) * P;
    const int rows = (N + SS_PARTS - 1) / SS_PARTS;
    float s[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int i = part + SS_PARTS * j;
        s[j] = (j < rows && i < N && col_ok) ? S[(size_t)i * P + col] : 0.f;
    }
    const float a = -expf(A_log[h]), bias = dt_bias[h], dskip = Dskip[h];
    const int ROW = 2 * N + SS_COLS + 1, ROWS = ROW + 1, EB = SS_TB * ROW;
    auto fetch = [&](int e, int tb0, int nb) -> float {          // element e of the batch of nb tokens that starts at token tb0
        const int tt = e / ROW, k = e - tt * ROW;
        if (tt >= nb) return 0.f;
        const size_t t = (size_t)(t0 + tb0 + tt);
        if (k < N) return to_f32<T>(xbc[t * C_ + inner + g * N + k]);
        if (k < 2 * N) return to_f32<T>(xbc[t * C_ + inner + groups * N + g * N + (k - N)]);
        if (k < 2 * N + SS_COLS) {
            const int c = col0 + k - 2 * N;
            return c < P ? to_f32<T>(xbc[t * C_ + h * P + c]) : 0.f;
        }
        return to_f32<T>(proj[t * stride + dt_off + h]);
    };
    auto put = [&](float* buf, int e, float v) {
        const int tt = e / ROW, k = e - tt * ROW;
        if (k < ROW - 1) {
            buf[tt * ROWS + k] = v;
        } else {
            const float dt = softplusf_(v + bias);
            buf[tt * ROWS + ROW - 1] = expf(a * dt);
            buf[tt * ROWS + ROW] = dt;
        }
    };
    const int n_batches = (n + SS_TB - 1) / SS_TB;
#pragma unroll
    for (int i = 0; i < PF; ++i) {
        const int e = tid + NT * i;
        if (e < EB) put(sm, e, fetch(e, 0, min(SS_TB, n)));
    }
    __syncthreads();
    for (int b = 0; b < n_batches; ++b) {
        const float* cur = sm + (b & 1) * SS_TB * ROWS;
        float* nxt = sm + ((b + 1) & 1) * SS_TB * ROWS;
        const bool more = b + 1 < n_batches;
        float pf[PF];
        if (more) {
            const int nb2 = min(SS_TB, n - (b + 1) * SS_TB);
#pragma unroll
            for (int i = 0; i < PF; ++i) {
                const int e = tid + NT * i;
                pf[i] = e < EB ? fetch(e, (b + 1) * SS_TB, nb2) : 0.f;
            }
        }
        const int nb = min(SS_TB, n - b * SS_TB);
        for (int tt = 0; tt < nb; ++tt) {
            const float* Bb = cur + tt * ROWS;
            const float* Cb = Bb + N;
            const float x = Bb[2 * N + (tid >> 3)], decay = Bb[ROW - 1], dx = Bb[ROW] * x;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < NR; ++j) {
                if (j < rows) {
                    const int i = part + SS_PARTS * j;
                    if (i < N) {
                        s[j] = fmaf(decay, s[j], Bb[i] * dx);
                        acc = fmaf(s[j], Cb[i], acc);
                    }
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (part == 0 && col_ok) y[(size_t)(t0 + b * SS_TB + tt) * inner + h * P + col] = acc + dskip * x;
        }
        if (more) {
#pragma unroll
            for (int i = 0; i < PF; ++i) {
                const int e = tid + NT * i;
                if (e < EB) put(nxt, e, pf[i]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int i = part + SS_PARTS * j;
        if (j < rows && i < N && col_ok) S[(size_t)i * P + col] = s[j];
    }
}

MSGL_API int msgl_ssm_scan(const void* xbc, int heads, int groups, int N, int P, const void* proj, long long stride, int dt_off,
                           const float* dt_bias, const float* A_log, const float* Dskip, float* state, const int* q_start,
                           const int* slots, float* y, int B, int dtype, cudaStream_t stream) {
    if (B <= 0) return MSGL_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0 || N > SS_PARTS * SS_MAX_ROWS) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const dim3 grid(B, heads, (P + SS_COLS - 1) / SS_COLS);
    const size_t smem = (size_t)2 * SS_TB * (2 * N + SS_COLS + 2) * sizeof(float);
    const int nr = (N + SS_PARTS - 1) / SS_PARTS;
#define SS_LAUNCH(NRR)                                                                                                          \
    do {                                                                                                                        \
        static MsglOncePerDevice once;                                                                                          \
        if (smem > 48 * 1024 && once.due()) {                                                                                   \
            cudaFuncSetAttribute(ssm_scan_kernel<float, NRR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);         \
            cudaFuncSetAttribute(ssm_scan_kernel<__nv_bfloat16, NRR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
            once.mark();                                                                                                        \
        }                                                                                                                       \
        if (dtype == MSGL_F32)                                                                                                  \
            ssm_scan_kernel<float, NRR><<<grid, SS_COLS * SS_PARTS, smem, stream>>>(xbc, heads, groups, N, P, proj, stride, dt_off, dt_bias, \
                                                                                  A_log, Dskip, state, q_start, slots, y);      \
        else                                                                                                                    \
            ssm_scan_kernel<__nv_bfloat16, NRR><<<grid, SS_COLS * SS_PARTS, smem, stream>>>(xbc, heads, groups, N, P, proj, stride, dt_off,  \
                                                                                          dt_bias, A_log, Dskip, state, q_start, slots, y); \
    } while (0)
    if (nr <= 4) SS_LAUNCH(4);
    else if (nr <= 8) SS_LAUNCH(8);
    else if (nr <= 16) SS_LAUNCH(16);
    else if (nr <= 32) SS_LAUNCH(32);
    else SS_LAUNCH(64);
#undef SS_LAUNCH
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// The state-space recurrence over long portions: the tokens of a request in chunks of SC_L that run side by side.  With
// la_t = the sum of log decay over the chunk's tokens up to and including t (log decay = -exp(A_log) * step, never positive):
//     S_t = exp(la_t) S_start + sum over j <= t of exp(la_t - la_j) step_j B_j x_j^T
// so a chunk is  S_end = exp(la_end) S_start + U  with  U = sum over t of exp(la_end - la_t) step_t B_t x_t^T, and
//     y_t = exp(la_t) S_start^T C_t + sum over j <= t of [exp(la_t - la_j) step_j (C_t . B_j)] x_j + D x_t.
// Every exponent is <= 0.  ssm_chunk_state_kernel leaves U and exp(la_end) of every (chunk, head); ssm_chunk_carry_kernel walks
// a request's chunks in order, replaces each U by the state at the chunk's start and writes the request's state back;
// ssm_chunk_out_kernel forms the outputs.  Float32 throughout; the result differs from the token-by-token kernel by rounding only.
// Grid: x = head * column tiles + column tile, y = chunk (over all requests, in order).
// ---------------------------------------------------------------------------------------
#define SC_L 64             // tokens of a chunk
#define SC_PT 64            // value columns of a block
#define SC_THREADS 256
#define SC_LS (SC_L + 4)    // row stride of the chunk's weights

// steps and running log decays of the chunk's n tokens (rows beyond n: step 0, the last token's sum)
template <typename T>
__device__ __forceinline__ void ssm_chunk_steps(const T* __restrict__ proj, long long stride, int col, int t0, int n, float bias, float a,
                                                float* dts, float* las) {
    const int tid = threadIdx.x;
    if (tid < SC_L) dts[tid] = tid < n ? softplusf_(to_f32<T>(proj[(size_t)(t0 + tid) * stride + col]) + bias) : 0.f;
    __syncthreads();
    if (tid < 32) {
        const float v0 = a * dts[2 * tid], v1 = v0 + a * dts[2 * tid + 1];
        float run = v1;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float o = __shfl_up_sync(0xffffffffu, run, d);
            if (tid >= d) run += o;
        }
        float before = __shfl_up_sync(0xffffffffu, run, 1);
        if (tid == 0) before = 0.f;
        las[2 * tid] = before + v0;
        las[2 * tid + 1] = before + v1;
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
ssm_chunk_state_kernel(const void* xbc_, int heads, int groups, int N, int P, const void* proj_, long long stride, int dt_off,
                       const float* __restrict__ dt_bias, const float* __restrict__ A_log, const int* __restrict__ q_start, int B,
                       float* __restrict__ U, float* __restrict__ Adec) {
    extern __shared__ __align__(16) float sc_sm[];
    __shared__ int sh[3];
    __shared__ float dts[SC_L], las[SC_L], ws[SC_L];
    int r, first, ci;
    if (!find_chunk_y(q_start, B, SC_L, sh, r, first, ci)) return;
    const int ptiles = (P + SC_PT - 1) / SC_PT;
    const int h = blockIdx.x / ptiles, p0 = (blockIdx.x - h * ptiles) * SC_PT;
    const int tid = threadIdx.x;
    const int t0 = q_start[r] + ci * SC_L, n = min(SC_L, q_start[r + 1] - t0);
    const int g = h / (heads / groups), inner = heads * P, C_ = inner + 2 * groups * N;
    const int NP = (N + 7) & ~7, NS = NP + 4;
    float* Bw = sc_sm;                   // [SC_L][NS]: B_t * exp(la_end - la_t) * step_t
    float* xs = sc_sm + SC_L * NS;       // [SC_L][SC_PT]
    const T* xbc = reinterpret_cast<const T*>(xbc_);
    ssm_chunk_steps<T>(reinterpret_cast<const T*>(proj_), stride, dt_off + h, t0, n, dt_bias[h], -expf(A_log[h]), dts, las);
    const float la_end = las[SC_L - 1];
    if (tid < SC_L) ws[tid] = expf(la_end - las[tid]) * dts[tid];
    __syncthreads();
    for (int e = tid; e < SC_L * NP; e += SC_THREADS) {
        const int t = e / NP, k = e - t * NP;
        Bw[t * NS + k] = (t < n && k < N) ? to_f32<T>(xbc[(size_t)(t0 + t) * C_ + inner + g * N + k]) * ws[t] : 0.f;
    }
    for (int e = tid; e < SC_L * SC_PT; e += SC_THREADS) {
        const int t = e / SC_PT, p = p0 + (e - t * SC_PT);
        xs[e] = (t < n && p < P) ? to_f32<T>(xbc[(size_t)(t0 + t) * C_ + h * P + p]) : 0.f;
    }
    __syncthreads();
    const int tn = tid >> 4, tp = tid & 15;
    float* Uo = U + (((size_t)(first + ci) * heads + h) * N) * P;
    const bool vec = (P & 3) == 0;
    for (int nb = 0; nb < NP; nb += 128) {
        const int n0 = nb + tn * 8;
        if (n0 >= NP) continue;
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll 2
        for (int t = 0; t < n; ++t) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + t * SC_PT + tp * 4);
            const float4 b0 = *reinterpret_cast<const float4*>(Bw + t * NS + n0);
            const float4 b1 = *reinterpret_cast<const float4*>(Bw + t * NS + n0 + 4);
            const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                acc[i][0] = fmaf(bb[i], xv.x, acc[i][0]);
                acc[i][1] = fmaf(bb[i], xv.y, acc[i][1]);
                acc[i][2] = fmaf(bb[i], xv.z, acc[i][2]);
                acc[i][3] = fmaf(bb[i], xv.w, acc[i][3]);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int k = n0 + i, p = p0 + tp * 4;
            if (k >= N || p >= P) continue;
            float* o = Uo + (size_t)k * P + p;
            if (vec) {
                *reinterpret_cast<float4*>(o) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (p + q < P) o[q] = acc[i][q];
            }
        }
    }
    if (tid == 0 && p0 == 0) Adec[(size_t)(first + ci) * heads + h] = expf(la_end);
}

// U [chunk][head][N * P]: in, a chunk's own sum; out, the state at the chunk's start.  Thread = one state element of (request, head).
__global__ void ssm_chunk_carry_kernel(int heads, int NPel, const int* __restrict__ q_start, const int* __restrict__ slots,
                                       float* __restrict__ U, const float* __restrict__ Adec, float* __restrict__ state) {
    const int r = blockIdx.z, h = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= NPel) return;
    int first = 0;
    for (int q = 0; q < r; ++q) first += (q_start[q + 1] - q_start[q] + SC_L - 1) / SC_L;
    const int nc = (q_start[r + 1] - q_start[r] + SC_L - 1) / SC_L;
    if (nc <= 0) return;
    float* Sg = state + ((size_t)slots[r] * heads + h) * NPel + e;
    float S = *Sg;
    const size_t step = (size_t)heads * NPel;
    size_t idx = ((size_t)first * heads + h) * NPel + e;
    for (int c0 = 0; c0 < nc; c0 += 8) {                 // eight chunks' reads in flight, then their updates in order
        float own[8], dec[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c0 + i < nc) {
                own[i] = U[idx + i * step];
                dec[i] = Adec[(size_t)(first + c0 + i) * heads + h];
            }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (c0 + i < nc) {
                U[idx + i * step] = S;
                S = fmaf(dec[i], S, own[i]);
            }
        idx += 8 * step;
    }
    *Sg = S;
}

template <typename T>
__global__ void __launch_bounds__(SC_THREADS)
ssm_chunk_out_kernel(const void* xbc_, int heads, int groups, int N, int P, const void* proj_, long long stride, int dt_off,
                     const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
                     const int* __restrict__ q_start, int B, const float* __restrict__ U, float* __restrict__ y) {
    extern __shared__ __align__(16) float sc_sm[];
    __shared__ int sh[3];
    __shared__ float dts[SC_L], las[SC_L];
    int r, first, ci;
    if (!find_chunk_y(q_start, B, SC_L, sh, r, first, ci)) return;
    const int ptiles = (P + SC_PT - 1) / SC_PT;
    const int h = blockIdx.x / ptiles, p0 = (blockIdx.x - h * ptiles) * SC_PT;
    const int tid = threadIdx.x;
    const int t0 = q_start[r] + ci * SC_L, n = min(SC_L, q_start[r + 1] - t0);
    const int g = h / (heads / groups), inner = heads * P, C_ = inner + 2 * groups * N;
    const int NP = (N + 7) & ~7, NS = NP + 4;
    float* Cs = sc_sm;                       // [SC_L][NS]
    float* Bs = Cs + SC_L * NS;              // [SC_L][NS]
    float* xs = Bs + SC_L * NS;              // [SC_L][SC_PT]
    float* Ws = xs + SC_L * SC_PT;           // [SC_L][SC_LS]: weight of token j's x in token t's output
    const T* xbc = reinterpret_cast<const T*>(xbc_);
    ssm_chunk_steps<T>(reinterpret_cast<const T*>(proj_), stride, dt_off + h, t0, n, dt_bias[h], -expf(A_log[h]), dts, las);
    for (int e = tid; e < SC_L * NP; e += SC_THREADS) {
        const int t = e / NP, k = e - t * NP;
        const bool ok = t < n && k < N;
        const size_t at = (size_t)(t0 + t) * C_ + inner + g * N + k;
        Bs[t * NS + k] = ok ? to_f32<T>(xbc[at]) : 0.f;
        Cs[t * NS + k] = ok ? to_f32<T>(xbc[at + (size_t)groups * N]) : 0.f;
    }
    for (int e = tid; e < SC_L * SC_PT; e += SC_THREADS) {
        const int t = e / SC_PT, p = p0 + (e - t * SC_PT);
        xs[e] = (t < n && p < P) ? to_f32<T>(xbc[(size_t)(t0 + t) * C_ + h * P + p]) : 0.f;
    }
    __syncthreads();
    const int ti = tid >> 4, tj = tid & 15;
    {   // C_t . B_j for the 4 x 4 pairs t = ti + 16 a, j = tj + 16 b
        float gacc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a) gacc[a][0] = gacc[a][1] = gacc[a][2] = gacc[a][3] = 0.f;
        for (int k = 0; k < NP; k += 4) {
            float4 c[4], b[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                c[a] = *reinterpret_cast<const float4*>(Cs + (ti + 16 * a) * NS + k);
                b[a] = *reinterpret_cast<const float4*>(Bs + (tj + 16 * a) * NS + k);
            }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int bq = 0; bq < 4; ++bq)
                    gacc[a][bq] = fmaf(c[a].w, b[bq].w, fmaf(c[a].z, b[bq].z, fmaf(c[a].y, b[bq].y, fmaf(c[a].x, b[bq].x, gacc[a][bq]))));
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int bq = 0; bq < 4; ++bq) {
                const int t = ti + 16 * a, j = tj + 16 * bq;
                Ws[t * SC_LS + j] = (j <= t && t < n) ? gacc[a][bq] * (expf(las[t] - las[j]) * dts[j]) : 0.f;
            }
    }
    __syncthreads();
    const int tp = tj;
    float acc[4][4], acs[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
        acs[a][0] = acs[a][1] = acs[a][2] = acs[a][3] = 0.f;
    }
#pragma unroll 2
    for (int j = 0; j < n; ++j) {
        const float4 xv = *reinterpret_cast<const float4*>(xs + j * SC_PT + tp * 4);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const float w = Ws[(ti + 16 * a) * SC_LS + j];
            acc[a][0] = fmaf(w, xv.x, acc[a][0]);
            acc[a][1] = fmaf(w, xv.y, acc[a][1]);
            acc[a][2] = fmaf(w, xv.z, acc[a][2]);
            acc[a][3] = fmaf(w, xv.w, acc[a][3]);
        }
    }
    // the state at the chunk's start goes through the shared memory that held B (N * SC_PT <= SC_L * NS floats)
    const float* S = U + (((size_t)(first + ci) * heads + h) * N) * P;
    float* Ss = Bs;                          // [N][SC_PT], zero beyond the head's columns
    const bool vec = (P & 3) == 0;
    if (vec) {
        for (int e = tid; e < N * (SC_PT / 4); e += SC_THREADS) {
            const int k = e / (SC_PT / 4), q = (e - k * (SC_PT / 4)) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p0 + q < P) v = *reinterpret_cast<const float4*>(S + (size_t)k * P + p0 + q);
            *reinterpret_cast<float4*>(Ss + k * SC_PT + q) = v;
        }
    } else {
        for (int e = tid; e < N * SC_PT; e += SC_THREADS) {
            const int k = e / SC_PT, q = e - k * SC_PT;
            Ss[e] = p0 + q < P ? S[(size_t)k * P + p0 + q] : 0.f;
        }
    }
    __syncthreads();
    const int pc = p0 + tp * 4;
    if (pc < P) {
#pragma unroll 4
        for (int k = 0; k < N; ++k) {
            const float4 sv = *reinterpret_cast<const float4*>(Ss + k * SC_PT + tp * 4);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float c = Cs[(ti + 16 * a) * NS + k];
                acs[a][0] = fmaf(c, sv.x, acs[a][0]);
                acs[a][1] = fmaf(c, sv.y, acs[a][1]);
                acs[a][2] = fmaf(c, sv.z, acs[a][2]);
                acs[a][3] = fmaf(c, sv.w, acs[a][3]);
            }
        }
        const float dskip = Dskip[h];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const int t = ti + 16 * a;
            if (t >= n) continue;
            const float e = expf(las[t]);
            float* o = y + (size_t)(t0 + t) * inner + h * P + pc;
            const float* xr = xs + t * SC_PT + tp * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (pc + q < P) o[q] = fmaf(e, acs[a][q], acc[a][q]) + dskip * xr[q];
        }
    }
}

// n_chunks: the sum over the requests of ceil(tokens / SC_L); U: float32 [n_chunks][heads][N][P] (16-byte aligned); Adec: float32
// [n_chunks][heads]
MSGL_API int msgl_ssm_scan_chunked(const void* xbc, int heads, int groups, int N, int P, const void* proj, long long stride, int dt_off,
                                   const float* dt_bias, const float* A_log, const float* Dskip, float* state, const int* q_start,
                                   const int* slots, float* y, int B, int n_chunks, float* U, float* Adec, int dtype, cudaStream_t stream) {
    if (B <= 0 || n_chunks <= 0) return MSGL_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0 || U == nullptr || Adec == nullptr || n_chunks > 65535 ||
        B > 65535 || heads > 65535 || ((uintptr_t)U & 15))
        return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const int NS = ((N + 7) & ~7) + 4;
    const size_t smem_state = (size_t)(SC_L * NS + SC_L * SC_PT) * sizeof(float);
    const size_t smem_out = (size_t)(2 * SC_L * NS + SC_L * SC_PT + SC_L * SC_LS) * sizeof(float);
    const size_t smem_max = 200 * 1024;
    if (smem_out > smem_max) return MSGL_ERR_SIZE;
    static MsglOncePerDevice once;
    if (once.due()) {
        cudaFuncSetAttribute(ssm_chunk_state_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max);
        cudaFuncSetAttribute(ssm_chunk_state_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max);
        cudaFuncSetAttribute(ssm_chunk_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max);
        cudaFuncSetAttribute(ssm_chunk_out_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max);
        once.mark();
    }
    const int ptiles = (P + SC_PT - 1) / SC_PT;
    const dim3 grid(heads * ptiles, n_chunks);
    const int NPel = N * P;
    const dim3 cgrid((NPel + 255) / 256, heads, B);
    if (dtype == MSGL_F32) {
        ssm_chunk_state_kernel<float><<<grid, SC_THREADS, smem_state, stream>>>(xbc, heads, groups, N, P, proj, stride, dt_off, dt_bias, A_log,
                                                                              q_start, B, U, Adec);
        ssm_chunk_carry_kernel<<<cgrid, 256, 0, stream>>>(heads, NPel, q_start, slots, U, Adec, state);
        ssm_chunk_out_kernel<float><<<grid, SC_THREADS, smem_out, stream>>>(xbc, heads, groups, N, P, proj, stride, dt_off, dt_bias, A_log,
                                                                          Dskip, q_start, B, U, y);
    } else {
        ssm_chunk_state_kernel<__nv_bfloat16><<<grid, SC_THREADS, smem_state, stream>>>(xbc, heads, groups, N, P, proj, stride, dt_off, dt_bias,
                                                                                      A_log, q_start, B, U, Adec);
        ssm_chunk_carry_kernel<<<cgrid, 256, 0, stream>>>(heads, NPel, q_start, slots, U, Adec, state);
        ssm_chunk_out_kernel<__nv_bfloat16><<<grid, SC_THREADS, smem_out, stream>>>(xbc, heads, groups, N, P, proj, stride, dt_off, dt_bias,
                                                                                  A_log, Dskip, q_start, B, U, y);
    }
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// out = (y * silu(z)) / rms over each of `parts` equal parts of the row * w * c:  the gate comes BEFORE the norm
//   y float32 [T, N] contiguous; z and out [T, N] views into packed rows of the activation type; w float32 [N]
// One warp per (token, part).
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void gate_group_norm_kernel(const float* __restrict__ y, int N, int parts, const float* __restrict__ w, float eps,
                                       const void* z_, long long z_stride, void* out_, long long out_stride, float c, int T_) {
    const long long wi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (wi >= (long long)T_ * parts) return;
    const int t = (int)(wi / parts), g = (int)(wi - (long long)t * parts);
    const int n = N / parts;
    const float* yr = y + (size_t)t * N + (size_t)g * n;
    const T* zr = reinterpret_cast<const T*>(z_) + (size_t)t * z_stride + (size_t)g * n;
    T* orow = reinterpret_cast<T*>(out_) + (size_t)t * out_stride + (size_t)g * n;
    float ss = 0.f;
#pragma unroll 8
    for (int i = lane; i < n; i += 32) { const float v = yr[i] * siluf_(to_f32<T>(zr[i])); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float f = rsqrtf(ss / (float)n + eps) * c;
#pragma unroll 8
    for (int i = lane; i < n; i += 32)
        orow[i] = from_f32<T>(yr[i] * siluf_(to_f32<T>(zr[i])) * f * w[(size_t)g * n + i]);
}

MSGL_API int msgl_gate_group_norm(const float* y, int N, int parts, const float* w, float eps, const void* z, long long z_stride,
                                  void* out, long long out_stride, float c, int T_, int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (N <= 0 || parts <= 0 || N % parts) return MSGL_ERR_SIZE;
    const long long warps = (long long)T_ * parts;
    const unsigned grid = (unsigned)((warps + 7) / 8);
    if (dtype == MSGL_F32) gate_group_norm_kernel<float><<<grid, 256, 0, stream>>>(y, N, parts, w, eps, z, z_stride, out, out_stride, c, T_);
    else if (dtype == MSGL_BF16) gate_group_norm_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(y, N, parts, w, eps, z, z_stride, out, out_stride, c, T_);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// out = act(x) * c, act: 0 silu, 1 gelu_tanh, 2 sigmoid, 3 relu(x)^2, 4 relu; [T, N] views with row strides of their own
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void unary_act_kernel(const T* __restrict__ x, long long x_stride, T* __restrict__ out, long long out_stride, int N, int act, float c) {
    const size_t t = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x) {
        out[t * out_stride + i] = from_f32<T>(act_of(act, to_f32<T>(x[t * x_stride + i])) * c);
    }
}

// 16 bytes a thread over the flattened [T, N / V] grid
template <typename T>
__global__ void __launch_bounds__(256) unary_act_vec_kernel(const T* __restrict__ x, long long x_stride, T* __restrict__ out,
                                                            long long out_stride, int N, int act, float c, long long total) {
    constexpr int V = VecOf<T>::N;
    const int per = N / V;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long t = e / per;
        const int i = (int)(e - t * per) * V;
        float v[V];
        VecOf<T>::load(x + t * x_stride + i, v);
#pragma unroll
        for (int k = 0; k < V; ++k) v[k] = act_of(act, v[k]) * c;
        VecOf<T>::store(out + t * out_stride + i, v);
    }
}

MSGL_API int msgl_unary_act(const void* x, long long x_stride, void* out, long long out_stride, int N, int act, float c, int T_, int dtype,
                            cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (N <= 0 || act < 0 || act > 4) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const int V = dtype == MSGL_F32 ? 4 : 8;
    if (N % V == 0 && x_stride % V == 0 && out_stride % V == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const long long total = (long long)T_ * (N / V);
        const int blocks = (int)min((total + 255) / 256, (long long)msgl_sm_count() * 16);
        if (dtype == MSGL_F32) unary_act_vec_kernel<float><<<blocks, 256, 0, stream>>>((const float*)x, x_stride, (float*)out, out_stride, N, act, c, total);
        else unary_act_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, x_stride, (__nv_bfloat16*)out, out_stride, N, act, c, total);
        return msgl_check_launch();
    }
    const dim3 grid(max(1, min((N + 255) / 256, 64)), T_);
    if (dtype == MSGL_F32) unary_act_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, x_stride, (float*)out, out_stride, N, act, c);
    else if (dtype == MSGL_BF16) unary_act_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, x_stride, (__nv_bfloat16*)out, out_stride, N, act, c);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Router of a mixture of experts: one block per token
//
//   z = W h (float32 sums), s = sigmoid(z), choice = s + correction
//   the experts form `n_groups` equal groups of neighbours; a group's score is the sum of its two largest choice scores; only
//   experts of the `keep` best groups can be chosen; the `top` largest choice scores among them are chosen (the lower index
//   wins a tie); weights = the chosen experts' s over their sum (+ 1e-20)
//   -> idx int32 [T, top], wts float32 [T, top]
// ---------------------------------------------------------------------------------------
#define RT_MAX_EXPERTS 1024
#define RT_MAX_GROUPS 64
template <typename T>
__global__ void __launch_bounds__(256) route_kernel(const T* __restrict__ h, long long h_stride, const T* __restrict__ W,
                                                    const float* __restrict__ correction, int H, int E, int n_groups, int keep,
                                                    int top, int* __restrict__ idx, float* __restrict__ wts, int vec, int softmax,
                                                    const T* __restrict__ gate_row, float* __restrict__ gate_out) {
    __shared__ float s_sh[RT_MAX_EXPERTS], c_sh[RT_MAX_EXPERTS], g_sh[RT_MAX_GROUPS];
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const T* hr = h + (size_t)t * h_stride;
    // row E, if there is one, is no expert: the sigmoid of its product with the token is handed out beside the choice
    for (int e = warp; e < E + (gate_row ? 1 : 0); e += nw) {
        const T* wr = e < E ? W + (size_t)e * H : gate_row;
        float acc = 0.f;
        if (vec) {                                       // 16 bytes of the row a lane and turn
            constexpr int V = VecOf<T>::N;
#pragma unroll 2
            for (int i = lane * V; i < H; i += 32 * V) {
                float a[V], b[V];
                VecOf<T>::load(wr + i, a);
                VecOf<T>::load(hr + i, b);
#pragma unroll
                for (int k = 0; k < V; ++k) acc = fmaf(a[k], b[k], acc);
            }
        } else {
            for (int i = lane; i < H; i += 32) acc = fmaf(to_f32<T>(wr[i]), to_f32<T>(hr[i]), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (e >= E) {
                gate_out[t] = sigmoidf_(acc);
            } else if (softmax) {                        // the logits themselves are chosen by and weighted
                s_sh[e] = acc;
                c_sh[e] = acc;
            } else {
                const float s = sigmoidf_(acc);
                s_sh[e] = s;
                c_sh[e] = s + (correction ? correction[e] : 0.f);
            }
        }
    }
    __syncthreads();
    const int per = E / n_groups;
    if (keep < n_groups) {
        for (int g = tid; g < n_groups; g += blockDim.x) {
            float m1 = -INFINITY, m2 = -INFINITY;
            for (int i = 0; i < per; ++i) {
                const float v = c_sh[g * per + i];
                if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) m2 = v;
            }
            g_sh[g] = per >= 2 ? m1 + m2 : m1;
        }
        __syncthreads();
        if (tid == 0) {
            // the groups that are not among the `keep` best lose their experts
            for (int k = 0; k < keep; ++k) {
                int best = -1; float bv = -INFINITY;
                for (int g = 0; g < n_groups; ++g)
                    if (!isnan(g_sh[g]) && (best < 0 || g_sh[g] > bv)) { best = g; bv = g_sh[g]; }
                if (best >= 0) g_sh[best] = NAN;          // taken
            }
        }
        __syncthreads();
        for (int e = tid; e < E; e += blockDim.x)
            if (!isnan(g_sh[e / per])) c_sh[e] = -INFINITY;
        __syncthreads();
    }
    if (warp == 0) {
        float total = 0.f, first = 0.f;
        for (int k = 0; k < top; ++k) {
            float bv = -INFINITY; int be = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float v = c_sh[e];
                if (!isnan(v) && (v > bv || (v == bv && e < be))) { bv = v; be = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oe = __shfl_xor_sync(0xffffffffu, be, o);
                if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
            }
            if (be >= E) be = 0;                          // nothing left to choose from (top > experts allowed): refused on the host
            if (lane == 0) { idx[(size_t)t * top + k] = be; c_sh[be] = NAN; }
            if (k == 0) first = s_sh[be];                 // the largest chosen logit: the softmax's reference
            total += softmax ? expf(s_sh[be] - first) : s_sh[be];
            __syncwarp();
        }
        if (softmax) {                                    // softmax over the chosen logits only
            const float inv = 1.f / total;
            for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] = expf(s_sh[idx[(size_t)t * top + k]] - first) * inv;
        } else {
            const float inv = 1.f / (total + 1e-20f);
            for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] = s_sh[idx[(size_t)t * top + k]] * inv;
        }
    }
}

MSGL_API int msgl_route(const void* h, long long h_stride, const void* W, const float* correction, int H, int E, int n_groups, int keep,
                        int top, int* idx, float* wts, int T_, int dtype, int softmax, const void* gate_row, float* gate_out,
                        cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (H <= 0 || E <= 0 || E > RT_MAX_EXPERTS || n_groups < 1 || n_groups > RT_MAX_GROUPS || E % n_groups || keep < 1 || keep > n_groups ||
        top < 1 || top > keep * (E / n_groups))
        return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    // whether rows can be read 16 bytes at a time: a matter of the sizes and of the weights' place, the same in every step of a model
    const int V = dtype == MSGL_F32 ? 4 : 8;
    const int vec = H % V == 0 && h_stride % V == 0 && ((uintptr_t)h % 16) == 0 && ((uintptr_t)W % 16) == 0 &&
                    ((uintptr_t)gate_row % 16) == 0;
    if (gate_row && !gate_out) return MSGL_ERR_SIZE;
    const int threads = E > 4 ? 256 : 128;
    if (dtype == MSGL_F32) route_kernel<float><<<T_, threads, 0, stream>>>((const float*)h, h_stride, (const float*)W, correction, H, E, n_groups, keep, top, idx, wts, vec, softmax, (const float*)gate_row, gate_out);
    else route_kernel<__nv_bfloat16><<<T_, threads, 0, stream>>>((const __nv_bfloat16*)h, h_stride, (const __nv_bfloat16*)W, correction, H, E, n_groups, keep, top, idx, wts, vec, softmax, (const __nv_bfloat16*)gate_row, gate_out);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// The chosen experts' products for a few tokens, straight from the stacked weights
//
//   act[t * top + k, r] = silu(Wg[e][r] . h_t) * (Wu[e][r] . h_t),  e = idx[t, k];   Wgu [E][2][F][H] = an expert's gate, then its up
//   out[t, c] = c_out * sum_k wts[t, k] * (Wd[e_k][c] . act[t * top + k, :]) in float32;   Wd [E][H][F]
// One warp per output row of a (token, choice) pair, resp. per output column of a token.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) expert_gate_up_kernel(const T* __restrict__ h, long long h_stride, const T* __restrict__ Wgu,
                                                             const int* __restrict__ idx, int top, int H, int F, T* __restrict__ act,
                                                             float limit) {
    const int pair = blockIdx.y, t = pair / top;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= F) return;
    const int e = idx[pair];
    const T* hr = h + (size_t)t * h_stride;
    const T* g = Wgu + ((size_t)e * 2 * F + r) * H;
    const T* u = g + (size_t)F * H;
    float ag = 0.f, au = 0.f;
    for (int i = lane; i < H; i += 32) {
        const float x = to_f32<T>(hr[i]);
        ag = fmaf(to_f32<T>(g[i]), x, ag);
        au = fmaf(to_f32<T>(u[i]), x, au);
    }
    ag = warp_sum(ag); au = warp_sum(au);
    if (lane == 0) act[(size_t)pair * F + r] = from_f32<T>(limit > 0.f ? clamped_gluf_(ag, au, limit) : siluf_(ag) * au);
}

template <typename T>
__global__ void __launch_bounds__(256) expert_down_kernel(const T* __restrict__ act, const T* __restrict__ Wd, const int* __restrict__ idx,
                                                          const float* __restrict__ wts, int top, int H, int F, float c_out,
                                                          float* __restrict__ out, const float* __restrict__ extra,
                                                          const float* __restrict__ extra_gate) {
    const int t = blockIdx.y;
    const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (c >= H) return;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const int e = idx[(size_t)t * top + k];
        const T* w = Wd + ((size_t)e * H + c) * F;
        const T* a = act + ((size_t)t * top + k) * F;
        float acc = 0.f;
        for (int i = lane; i < F; i += 32) acc = fmaf(to_f32<T>(w[i]), to_f32<T>(a[i]), acc);
        acc = warp_sum(acc);
        total = fmaf(wts[(size_t)t * top + k], acc, total);
    }
    if (lane == 0) {
        if (extra) total = fmaf(extra_gate ? extra_gate[t] : 1.f, extra[(size_t)t * H + c], total);
        out[(size_t)t * H + c] = total * c_out;
    }
}

MSGL_API int msgl_experts_few(const void* h, long long h_stride, const void* Wgu, const void* Wd, const int* idx,
                              const float* wts, int top, int H, int F, void* act, float c_out, float* out, int T_, int dtype,
                              float limit, const float* extra, const float* extra_gate, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (top < 1 || H <= 0 || F <= 0) return MSGL_ERR_SIZE;
    if (dtype != MSGL_F32 && dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    const dim3 g1((F + 7) / 8, T_ * top), g2((H + 7) / 8, T_);
    if (dtype == MSGL_F32) {
        expert_gate_up_kernel<float><<<g1, 256, 0, stream>>>((const float*)h, h_stride, (const float*)Wgu, idx, top, H, F, (float*)act, limit);
        expert_down_kernel<float><<<g2, 256, 0, stream>>>((const float*)act, (const float*)Wd, idx, wts, top, H, F, c_out, out, extra, extra_gate);
    } else {
        expert_gate_up_kernel<__nv_bfloat16><<<g1, 256, 0, stream>>>((const __nv_bfloat16*)h, h_stride, (const __nv_bfloat16*)Wgu, idx, top, H, F,
                                                                      (__nv_bfloat16*)act, limit);
        expert_down_kernel<__nv_bfloat16><<<g2, 256, 0, stream>>>((const __nv_bfloat16*)act, (const __nv_bfloat16*)Wd, idx, wts, top, H, F, c_out, out, extra, extra_gate);
    }
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Many tokens: the (token, choice) pairs in the order of their experts
//
//   expert_count_kernel   counts[e] = pairs whose expert is e                                   (one block per expert)
//   expert_place_kernel   place[pair] = row of the pair in expert order, stable within an expert  (one block per expert)
//   expert_gather_kernel  rows[place[pair]] = h[token of the pair]
//   expert_combine_kernel out[t] = c * sum_k wts[t, k] * y[place[t * top + k]] in float32
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) expert_count_kernel(const int* __restrict__ idx, int n_pairs, int* __restrict__ counts) {
    __shared__ float scratch[32];
    const int e = blockIdx.x;
    int n = 0;
    for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) n += idx[i] == e;
    const float total = block_sum((float)n, scratch);          // exact below 2^24 pairs
    if (threadIdx.x == 0) counts[e] = (int)(total + 0.5f);
}

__global__ void __launch_bounds__(256) expert_place_kernel(const int* __restrict__ idx, int n_pairs, const int* __restrict__ counts,
                                                           int* __restrict__ place) {
    __shared__ int warp_tot[8];
    __shared__ int base_sh;
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        int b = 0;
        for (int i = 0; i < e; ++i) b += counts[i];
        base_sh = b;
    }
    __syncthreads();
    int base = base_sh;
    for (int i0 = 0; i0 < n_pairs; i0 += 256) {
        const int i = i0 + tid;
        const bool mine = i < n_pairs && idx[i] == e;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_tot[warp] = __popc(m);
        __syncthreads();
        int before = 0, all = 0;
        for (int w = 0; w < 8; ++w) { if (w < warp) before += warp_tot[w]; all += warp_tot[w]; }
        if (mine) place[i] = base + before + __popc(m & ((1u << lane) - 1u));
        base += all;
        __syncthreads();
    }
}

template <typename T>
__global__ void expert_gather_kernel(const T* __restrict__ h, long long h_stride, const int* __restrict__ place, int top, int H,
                                     T* __restrict__ rows) {
    const int pair = blockIdx.x, t = pair / top;
    const T* src = h + (size_t)t * h_stride;
    T* dst = rows + (size_t)place[pair] * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
}

template <typename Y>
__global__ void expert_combine_kernel(const Y* __restrict__ y, const int* __restrict__ place, const float* __restrict__ wts, int top, int H,
                                      float c, float* __restrict__ out, const float* __restrict__ extra,
                                      const float* __restrict__ extra_gate) {
    const int t = blockIdx.x;
    const float eg = extra ? (extra_gate ? extra_gate[t] : 1.f) : 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) acc = fmaf(wts[(size_t)t * top + k], to_f32<Y>(y[(size_t)place[(size_t)t * top + k] * H + i]), acc);
        if (extra) acc = fmaf(eg, extra[(size_t)t * H + i], acc);
        out[(size_t)t * H + i] = acc * c;
    }
}

MSGL_API int msgl_expert_order(const int* idx, int n_pairs, int E, int* counts, int* place, cudaStream_t stream) {
    if (n_pairs <= 0) return MSGL_OK;
    if (E <= 0 || n_pairs >= (1 << 24)) return MSGL_ERR_SIZE;
    expert_count_kernel<<<E, 256, 0, stream>>>(idx, n_pairs, counts);
    expert_place_kernel<<<E, 256, 0, stream>>>(idx, n_pairs, counts, place);
    return msgl_check_launch();
}

MSGL_API int msgl_expert_gather(const void* h, long long h_stride, const int* place, int top, int H, void* rows, int n_pairs, int dtype,
                                cudaStream_t stream) {
    if (n_pairs <= 0) return MSGL_OK;
    if (dtype == MSGL_F32) expert_gather_kernel<float><<<n_pairs, 128, 0, stream>>>((const float*)h, h_stride, place, top, H, (float*)rows);
    else if (dtype == MSGL_BF16) expert_gather_kernel<__nv_bfloat16><<<n_pairs, 128, 0, stream>>>((const __nv_bfloat16*)h, h_stride, place, top, H, (__nv_bfloat16*)rows);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

MSGL_API int msgl_expert_combine(const void* y, int y_is_f32, const int* place, const float* wts, int top, int H, float c, float* out,
                                 int T_, const float* extra, const float* extra_gate, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (y_is_f32) expert_combine_kernel<float><<<T_, 256, 0, stream>>>((const float*)y, place, wts, top, H, c, out, extra, extra_gate);
    else expert_combine_kernel<__nv_bfloat16><<<T_, 256, 0, stream>>>((const __nv_bfloat16*)y, place, wts, top, H, c, out, extra, extra_gate);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Clamped gated activation of a packed [gate | up] row:  g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(1.702 g) * (u + 1), in float32, one thread per output element
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) clamped_glu_kernel(const T* __restrict__ gu, long long stride, int F, float limit,
                                                          T* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / F;
    const int c = (int)(i - t * F);
    const T* row = gu + t * stride;
    out[i] = from_f32<T>(clamped_gluf_(to_f32<T>(row[c]), to_f32<T>(row[F + c]), limit));
}

// the same, 16 bytes of gate and of up a thread
template <typename T>
__global__ void __launch_bounds__(256) clamped_glu_vec_kernel(const T* __restrict__ gu, long long stride, int F, float limit,
                                                              T* __restrict__ out, long long n_vec) {
    constexpr int V = VecOf<T>::N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const int per_row = F / V;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * V;
    float g[V], u[V], o[V];
    VecOf<T>::load(gu + t * stride + c, g);
    VecOf<T>::load(gu + t * stride + F + c, u);
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = clamped_gluf_(g[k], u[k], limit);
    VecOf<T>::store(out + t * F + c, o);
}

MSGL_API int msgl_clamped_glu(const void* gu, long long stride, int F, float limit, void* out, int T_, int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (F <= 0 || !(limit > 0.f)) return MSGL_ERR_SIZE;
    const int V = dtype == MSGL_F32 ? 4 : 8;
    if ((dtype == MSGL_F32 || dtype == MSGL_BF16) && F % V == 0 && stride % V == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const long long n_vec = (long long)T_ * (F / V);
        const unsigned vb = (unsigned)((n_vec + 255) / 256);
        if (dtype == MSGL_F32) clamped_glu_vec_kernel<float><<<vb, 256, 0, stream>>>((const float*)gu, stride, F, limit, (float*)out, n_vec);
        else clamped_glu_vec_kernel<__nv_bfloat16><<<vb, 256, 0, stream>>>((const __nv_bfloat16*)gu, stride, F, limit, (__nv_bfloat16*)out, n_vec);
        return msgl_check_launch();
    }
    const long long n = (long long)T_ * F;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == MSGL_F32) clamped_glu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, stride, F, limit, (float*)out, n);
    else if (dtype == MSGL_BF16) clamped_glu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, stride, F, limit, (__nv_bfloat16*)out, n);
    else return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}
