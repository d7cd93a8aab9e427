// linrec.cu -- linear-recurrence sequence mixers beside the selective scan of seqmix.cu:
//   (1) matrix-state recurrences with a decay per key channel: per head an fp32 state S [dk x dv] and, per token,
//           S <- diag(g_t) S ;  then either   S <- S + k_t v_t^T                                   (gated linear attention)
//                                     or      u = beta_t (v_t - S^T k_t),  S <- S + k_t u^T        (gated delta rule)
//       and the read-out o_t = S^T q_t, which sees the token's own write.  The decay is formed in fp32 from a logit z while the
//       token is staged: g = sigmoid(z + b)^(1/tau), or g = exp(-exp(A_h) softplus(z + b)).  q and k may be made unit vectors per head.
//   (2) a real-gated linear recurrent unit over channels: block-diagonal gate matmuls r, i = sigmoid(W u_b + b), decay
//       a = exp(-c r softplus(lam)), state s <- a s + sqrt(1 - a^2) i u, output s * y.
// State lives in fp32 per (sequence slot, layer) and persists between calls; a slot whose first staged token has position 0 starts
// from zero without a clearing pass.  Tokens are nseq sequences of T consecutive tokens (prefill panel 1 x M, batched decode M x 1).
// No reference equivalent (the reference's inference path is the Qwen3 attention block only).
#include <math.h>

#include <algorithm>

#include "kf_common.cuh"

namespace {
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

struct ScanArgs {
    float* y;          // [M][ldy] heads x dv
    int ldy;
    const float *q, *k, *v, *z, *beta;  // fp32 rows; q / k: kv-head major [G][dk]; v: [H][dv]; z: [H][dk]; beta logits [H] (delta only)
    int ldq, ldk, ldv, ldz, ldb;
    const uint16_t* zbias;   // bf16 [H * dk]
    const uint16_t* A_log;   // bf16 [H] (decay kind 1)
    float* state;            // [slot][H][dv][dk]
    size_t state_stride;
    const int32_t *pos, *slot;
    int T, H, G, dk, dv;
    int R, PB, TB;
    int delta;               // 1: delta-rule write, 0: plain outer-product write
    int decay_kind;          // 0: sigmoid(z + b)^(1/tau) ; 1: exp(-exp(A_h) softplus(z + b))
    int unit_qk;             // q, k divided by sqrt(sum x^2 + unit_eps) per head
    float inv_tau, q_scale, unit_eps;
};

// grid (heads, sequences, column chunks).  Thread (pl, r) keeps the NPT consecutive rows n = r * NPT + i of state column p0 + pl in
// registers (NPT = 16 / 32 / 64: up to 64 key channels sit in ONE thread, so that all lanes of a warp read the same k, q and decay
// entries -- one shared-memory broadcast per 16 bytes -- and nothing is reduced across lanes; larger key sizes use R = 2, 4, 8 adjacent
// lanes per column and shuffles).  TB tokens are staged in shared memory per pass: k, q (normalised there), the decay (formed there), v,
// beta.  FULL (dk == R * NPT): 16-byte shared loads and no bounds checks; otherwise rows beyond dk read k = q = 0 and keep a zero state.
template <bool DELTA, bool FULL, int NPT>
__global__ void __launch_bounds__(128) kf_gated_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int dk = a.dk, TB = a.TB, PB = a.PB, R = a.R;
    float* sK = sm;                  // [TB][dk]
    float* sQ = sK + TB * dk;        // [TB][dk]
    float* sG = sQ + TB * dk;        // [TB][dk]
    float* sV = sG + TB * dk;        // [TB][PB]
    float* sB = sV + TB * PB;        // [TB]
    const int h = blockIdx.x, seq = blockIdx.y, p0 = blockIdx.z * PB;
    const int kh = h / (a.H / a.G);
    const int tid = threadIdx.x, pl = tid / R, r = tid - pl * R, p = p0 + pl;
    const bool live = pl < PB && p < a.dv;
    const int m0 = seq * a.T, n0 = r * NPT;
    float* st = a.state + (size_t)a.slot[m0] * a.state_stride + ((size_t)h * a.dv + (live ? p : 0)) * dk;
    const bool fresh = a.pos[m0] == 0;
    float S[NPT];
#pragma unroll
    for (int i = 0; i < NPT; i++) S[i] = (live && n0 + i < dk && !fresh) ? st[n0 + i] : 0.f;
    const float Aexp = a.decay_kind == 1 ? expf(bf16_bits_to_f32(a.A_log[h])) : 0.f;
    const int warp = tid >> 5, lane = tid & 31, nwarp = blockDim.x >> 5;
    for (int t0 = 0; t0 < a.T; t0 += TB) {
        const int nt = min(TB, a.T - t0);
        __syncthreads();
        // four elements per thread and round: their global loads are issued together, then the decays are formed
        for (int i0 = tid; i0 < nt * dk; i0 += 4 * blockDim.x) {
            float kv[4], qv[4], zv[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = i0 + e * blockDim.x;
                if (i < nt * dk) {
                    const int tt = i / dk, n = i - tt * dk;
                    const size_t m = (size_t)(m0 + t0 + tt);
                    kv[e] = a.k[m * a.ldk + kh * dk + n], qv[e] = a.q[m * a.ldq + kh * dk + n];
                    zv[e] = a.z[m * a.ldz + h * dk + n] + (a.zbias ? bf16_bits_to_f32(a.zbias[h * dk + n]) : 0.f);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = i0 + e * blockDim.x;
                if (i < nt * dk) {
                    sK[i] = kv[e], sQ[i] = qv[e];
                    sG[i] = a.decay_kind == 1 ? expf(-Aexp * softplus_f(zv[e])) : expf(log_sigmoid_f(zv[e]) * a.inv_tau);
                }
            }
        }
        for (int i0 = tid; i0 < nt * PB; i0 += 4 * blockDim.x) {
            float vv[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = i0 + e * blockDim.x, tt = i / PB, c = i - tt * PB;
                vv[e] = (i < nt * PB && p0 + c < a.dv) ? a.v[(size_t)(m0 + t0 + tt) * a.ldv + h * a.dv + p0 + c] : 0.f;
            }
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (i0 + e * blockDim.x < nt * PB) sV[i0 + e * blockDim.x] = vv[e];
        }
        if (DELTA)
            for (int i = tid; i < nt; i += blockDim.x) sB[i] = sigmoid_f(a.beta[(size_t)(m0 + t0 + i) * a.ldb + h]);
        __syncthreads();
        // unit vectors / query scale: one warp per staged token
        for (int tt = warp; tt < nt; tt += nwarp) {
            float sq = 0.f, sk = 0.f;
            if (a.unit_qk) {
                for (int n = lane; n < dk; n += 32) sq = fmaf(sQ[tt * dk + n], sQ[tt * dk + n], sq), sk = fmaf(sK[tt * dk + n], sK[tt * dk + n], sk);
                sq = warp_sum(sq), sk = warp_sum(sk);
            }
            const float fq = a.unit_qk ? a.q_scale / sqrtf(sq + a.unit_eps) : a.q_scale;
            const float fk = a.unit_qk ? 1.f / sqrtf(sk + a.unit_eps) : 1.f;
            for (int n = lane; n < dk; n += 32) {
                sQ[tt * dk + n] *= fq;
                if (a.unit_qk) sK[tt * dk + n] *= fk;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float* kr = sK + tt * dk + n0;
            const float* qr = sQ + tt * dk + n0;
            const float* gr = sG + tt * dk + n0;
            // four entries of a staged row starting at row n0 + 4 j of this thread's slice
            auto ld4 = [&](const float* row, int j, float oob) -> float4 {
                if (FULL) return reinterpret_cast<const float4*>(row)[j];
                float4 v;
                v.x = n0 + 4 * j + 0 < dk ? row[4 * j + 0] : oob, v.y = n0 + 4 * j + 1 < dk ? row[4 * j + 1] : oob;
                v.z = n0 + 4 * j + 2 < dk ? row[4 * j + 2] : oob, v.w = n0 + 4 * j + 3 < dk ? row[4 * j + 3] : oob;
                return v;
            };
            const float vv = sV[tt * PB + (pl < PB ? pl : 0)];
            float w = vv;
            if (DELTA) {
                float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;  // four partial sums: short dependent chains
#pragma unroll
                for (int j = 0; j < NPT / 4; j++) {
                    const float4 gv = ld4(gr, j, 1.f), kv = ld4(kr, j, 0.f);
                    S[4 * j + 0] *= gv.x, S[4 * j + 1] *= gv.y, S[4 * j + 2] *= gv.z, S[4 * j + 3] *= gv.w;
                    d0 = fmaf(S[4 * j + 0], kv.x, d0), d1 = fmaf(S[4 * j + 1], kv.y, d1);
                    d2 = fmaf(S[4 * j + 2], kv.z, d2), d3 = fmaf(S[4 * j + 3], kv.w, d3);
                }
                float dot = (d0 + d1) + (d2 + d3);
                for (int o = R >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                w = sB[tt] * (vv - dot);
            }
            float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
            for (int j = 0; j < NPT / 4; j++) {
                const float4 kv = ld4(kr, j, 0.f), qv = ld4(qr, j, 0.f);
                if (DELTA) {
                    S[4 * j + 0] = fmaf(kv.x, w, S[4 * j + 0]), S[4 * j + 1] = fmaf(kv.y, w, S[4 * j + 1]);
                    S[4 * j + 2] = fmaf(kv.z, w, S[4 * j + 2]), S[4 * j + 3] = fmaf(kv.w, w, S[4 * j + 3]);
                } else {
                    const float4 gv = ld4(gr, j, 1.f);
                    S[4 * j + 0] = fmaf(gv.x, S[4 * j + 0], kv.x * w), S[4 * j + 1] = fmaf(gv.y, S[4 * j + 1], kv.y * w);
                    S[4 * j + 2] = fmaf(gv.z, S[4 * j + 2], kv.z * w), S[4 * j + 3] = fmaf(gv.w, S[4 * j + 3], kv.w * w);
                }
                c0 = fmaf(S[4 * j + 0], qv.x, c0), c1 = fmaf(S[4 * j + 1], qv.y, c1);
                c2 = fmaf(S[4 * j + 2], qv.z, c2), c3 = fmaf(S[4 * j + 3], qv.w, c3);
            }
            float acc = (c0 + c1) + (c2 + c3);
            for (int o = R >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && r == 0) a.y[(size_t)(m0 + t0 + tt) * a.ldy + h * a.dv + p] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPT; i++)
            if (n0 + i < dk) st[n0 + i] = S[i];
    }
}

// ------------------------------------------------------------------------------------------------------------ real-gated LRU
// Gates of TT tokens x 128 output channels of one block b:  r = sigmoid(Wr[b] u_b + br), i = sigmoid(Wi[b] u_b + bi), fp32 FMAs over
// the bf16 weights (staged transposed through shared memory so that every weight is read once per TT tokens); then
//   a = exp(-c r softplus(lam)),  A[m][ch] = a,  Bv[m][ch] = sqrt(1 - a^2) i u.
constexpr int GT = 8;
__global__ void __launch_bounds__(128) kf_rglru_gates_kernel(float* __restrict__ A, float* __restrict__ Bv, const float* __restrict__ u, int ldu,
                                                             const uint16_t* __restrict__ Wr, const uint16_t* __restrict__ br, const uint16_t* __restrict__ Wi,
                                                             const uint16_t* __restrict__ bi, const uint16_t* __restrict__ lam, int M, int width, int bs,
                                                             float c) {
    __shared__ float su[GT][32];
    __shared__ float swr[32][129], swi[32][129];
    const int m0 = blockIdx.x * GT, b = blockIdx.y, o0 = blockIdx.z * 128, o = o0 + threadIdx.x;
    const int nt = min(GT, M - m0);
    const uint16_t* wr = Wr + (size_t)b * bs * bs;
    const uint16_t* wi = Wi + (size_t)b * bs * bs;
    float ar[GT], ai[GT];
#pragma unroll
    for (int t = 0; t < GT; t++) ar[t] = ai[t] = 0.f;
    for (int i0 = 0; i0 < bs; i0 += 32) {
        __syncthreads();
        for (int e = threadIdx.x; e < 128 * 32; e += 128) {
            const int oo = e >> 5, ii = e & 31;
            const bool ok = o0 + oo < bs && i0 + ii < bs;
            swr[ii][oo] = ok ? bf16_bits_to_f32(wr[(size_t)(o0 + oo) * bs + i0 + ii]) : 0.f;
            swi[ii][oo] = ok ? bf16_bits_to_f32(wi[(size_t)(o0 + oo) * bs + i0 + ii]) : 0.f;
        }
        for (int e = threadIdx.x; e < GT * 32; e += 128) {
            const int t = e >> 5, ii = e & 31;
            su[t][ii] = (t < nt && i0 + ii < bs) ? u[(size_t)(m0 + t) * ldu + b * bs + i0 + ii] : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int ii = 0; ii < 32; ii++) {
            const float w1 = swr[ii][threadIdx.x], w2 = swi[ii][threadIdx.x];
#pragma unroll
            for (int t = 0; t < GT; t++) ar[t] = fmaf(w1, su[t][ii], ar[t]), ai[t] = fmaf(w2, su[t][ii], ai[t]);
        }
    }
    if (o >= bs) return;
    const int ch = b * bs + o;
    const float sp = softplus_f(bf16_bits_to_f32(lam[ch])), b1 = bf16_bits_to_f32(br[ch]), b2 = bf16_bits_to_f32(bi[ch]);
#pragma unroll
    for (int t = 0; t < GT; t++) {
        if (t >= nt) break;
        const float rg = sigmoid_f(ar[t] + b1), ig = sigmoid_f(ai[t] + b2);
        const float la = -c * rg * sp;
        const size_t m = (size_t)(m0 + t);
        A[m * width + ch]  = expf(la);
        Bv[m * width + ch] = sqrtf(-expm1f(2.f * la)) * ig * u[m * ldu + ch];
    }
}
// s <- A s + Bv along the T tokens of a sequence, out = s * gelu_tanh(y + yb) in the activation type.  A CTA owns 32 channels (one per
// lane) and its W warps each a run of consecutive tokens: a first pass reduces every run to one affine map s -> P s + B, the maps of the
// earlier runs give a warp its incoming state, a second pass replays the run and writes.  Loads are 128-byte rows across the lanes.
constexpr int LRU_W = 16;
template <typename TO>
__global__ void __launch_bounds__(32 * LRU_W) kf_rglru_scan_kernel(TO* __restrict__ out, int ldo, const float* __restrict__ A, const float* __restrict__ Bv,
                                                                   const float* __restrict__ y, int ldy, const uint16_t* __restrict__ yb,
                                                                   float* __restrict__ state, size_t state_stride, const int32_t* __restrict__ pos,
                                                                   const int32_t* __restrict__ slot, int T, int width) {
    __shared__ float sP[LRU_W][32], sB[LRU_W][32];
    const int seq = blockIdx.y, lane = threadIdx.x & 31, w = threadIdx.x >> 5, W = blockDim.x >> 5;
    const int ch = blockIdx.x * 32 + lane, m0 = seq * T;
    const bool live = ch < width;
    const int run = (T + W - 1) / W, t_lo = min(T, w * run), t_hi = min(T, t_lo + run);
    float* st = state + (size_t)slot[m0] * state_stride + (live ? ch : 0);
    float s = (pos[m0] == 0 || !live) ? 0.f : *st;
    float P = 1.f, B = 0.f;
    if (W > 1 && live) {
#pragma unroll 4
        for (int t = t_lo; t < t_hi; t++) {
            const size_t m = (size_t)(m0 + t);
            const float av = A[m * width + ch];
            B = fmaf(av, B, Bv[m * width + ch]);
            P *= av;
        }
    }
    sP[w][lane] = P, sB[w][lane] = B;
    __syncthreads();
    for (int q = 0; q < w; q++) s = fmaf(sP[q][lane], s, sB[q][lane]);
    if (!live) return;
    const float bias = yb ? bf16_bits_to_f32(yb[ch]) : 0.f;
#pragma unroll 4
    for (int t = t_lo; t < t_hi; t++) {
        const size_t m = (size_t)(m0 + t);
        s = fmaf(A[m * width + ch], s, Bv[m * width + ch]);
        const float o = s * gelu_tanh_f(y[m * ldy + ch] + bias);
        if (sizeof(TO) == 2) ((uint16_t*)out)[m * ldo + ch] = f32_to_bf16_bits(o);
        else ((float*)out)[m * ldo + ch] = o;
    }
    if (w == W - 1) *st = s;  // the last run ends at token T - 1 (runs may be empty only at the end when T < W, which the launch rules out)
}
}  // namespace

// Matrix-state recurrence over nseq x T tokens (see the head of this file).  q, k: float rows with G kv heads of dk entries at row strides
// ldq / ldk; v: H heads of dv entries; z: decay logits H x dk (+ bf16 bias zbias or NULL); beta_logit: H per token (delta rule only).
// decay_kind 0: g = sigmoid(z + b)^(1/tau); 1: g = exp(-exp(A_log[h]) softplus(z + b)).  state: float [slot][H][dv][dk].
extern "C" int kf_gated_scan(kf_ctx* ctx, float* y, int ldy, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* z,
                             int ldz, const void* zbias_bf16, const void* A_log_bf16, const float* beta_logit, int ldb, float* state, size_t state_stride,
                             const int32_t* pos_dev, const int32_t* slot_dev, int nseq, int T, int H, int G, int dk, int dv, int delta, int decay_kind,
                             float tau, int unit_qk, float unit_eps, float q_scale) {
    if (!ctx || !y || !q || !k || !v || !z || !state || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, nseq >= 1 && T >= 1 && H >= 1 && G >= 1 && H % G == 0 && dk >= 1 && dv >= 1 && dk <= 512, "key size <= 512, kv heads divide heads");
    KF_REQUIRE(ctx, (!delta || beta_logit) && (decay_kind == 0 ? tau > 0.f : A_log_bf16 != nullptr) && state_stride >= (size_t)H * dk * dv, "arguments");
    ScanArgs a = {};
    a.y = y, a.ldy = ldy, a.q = q, a.k = k, a.v = v, a.z = z, a.beta = beta_logit, a.ldq = ldq, a.ldk = ldk, a.ldv = ldv, a.ldz = ldz, a.ldb = ldb;
    a.zbias = (const uint16_t*)zbias_bf16, a.A_log = (const uint16_t*)A_log_bf16, a.state = state, a.state_stride = state_stride;
    a.pos = pos_dev, a.slot = slot_dev, a.T = T, a.H = H, a.G = G, a.dk = dk, a.dv = dv, a.delta = delta, a.decay_kind = decay_kind;
    a.unit_qk = unit_qk, a.inv_tau = decay_kind == 0 ? 1.f / tau : 0.f, a.q_scale = q_scale, a.unit_eps = unit_eps;
    // rows per thread: the whole key size when it is at most 64 (no lanes to reduce over), else 64 rows in each of R = 2, 4, 8 lanes
    const int NPT = dk <= 16 ? 16 : dk <= 32 ? 32 : 64;
    int R = 1;
    while (R * NPT < dk) R <<= 1;
    // up to 128 threads per CTA: the per-token chain of a warp is latency-bound and as long whatever the grid, while the staging of a pass
    // (and the decay's exponentials, formed once per CTA) is shared by the CTA's columns -- so columns are NOT spread over more, thinner CTAs
    const int PB = std::max(1, std::min(dv, 128 / R));
    const int threads = std::max(32, ((PB * R + 31) / 32) * 32);
    int TB = (int)std::min<size_t>(32, (44 * 1024 / sizeof(float)) / (size_t)(3 * dk + PB + 1));
    TB = std::max(1, std::min(TB, T));
    const size_t smem = (size_t)(3 * TB * dk + TB * PB + TB) * sizeof(float);
    KF_REQUIRE(ctx, smem <= 48 * 1024, "staging area");
    a.R = R, a.PB = PB, a.TB = TB;
    const dim3 grid(H, nseq, (dv + PB - 1) / PB);
    const bool full = dk == R * NPT;
#define KF_GS(D, F, N) kf_gated_scan_kernel<D, F, N><<<grid, threads, smem, ctx->stream>>>(a)
#define KF_GS_N(D, F) (NPT == 16 ? KF_GS(D, F, 16) : NPT == 32 ? KF_GS(D, F, 32) : KF_GS(D, F, 64))
    if (delta) {
        if (full) KF_GS_N(true, true);
        else KF_GS_N(true, false);
    } else {
        if (full) KF_GS_N(false, true);
        else KF_GS_N(false, false);
    }
#undef KF_GS_N
#undef KF_GS
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}

// Real-gated linear recurrent unit over `width` channels in `blocks` equal parts.  u: float [M][ldu] (the convolved branch); gate weights
// bf16 [blocks][bs][bs] ([out][in]) with biases [width]; lam bf16 [width]; y_logit: float [M][ldy] (+ bf16 bias), the other branch before
// its gelu.  out [M][ldo] = s * gelu_tanh(y) in the activation type.  work: float scratch [2][M][width].  state: float [slot][width].
extern "C" int kf_rglru(kf_ctx* ctx, void* out, int out_f32, int ldo, float* work, const float* u, int ldu, const void* w_r_bf16, const void* b_r_bf16,
                        const void* w_i_bf16, const void* b_i_bf16, const void* lam_bf16, float decay_c, const float* y_logit, int ldy,
                        const void* y_bias_bf16, float* state, size_t state_stride, const int32_t* pos_dev, const int32_t* slot_dev, int nseq, int T,
                        int width, int blocks) {
    if (!ctx || !out || !work || !u || !w_r_bf16 || !b_r_bf16 || !w_i_bf16 || !b_i_bf16 || !lam_bf16 || !y_logit || !state || !pos_dev || !slot_dev)
        return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, nseq >= 1 && T >= 1 && width >= 1 && blocks >= 1 && width % blocks == 0 && state_stride >= (size_t)width, "blocks must divide width");
    const int M = nseq * T, bs = width / blocks;
    float *A = work, *Bv = work + (size_t)M * width;
    kf_rglru_gates_kernel<<<dim3((M + GT - 1) / GT, blocks, (bs + 127) / 128), 128, 0, ctx->stream>>>(
        A, Bv, u, ldu, (const uint16_t*)w_r_bf16, (const uint16_t*)b_r_bf16, (const uint16_t*)w_i_bf16, (const uint16_t*)b_i_bf16, (const uint16_t*)lam_bf16, M,
        width, bs, decay_c);
    KF_LAUNCH_CHECK(ctx);
    dim3 grid((width + 31) / 32, nseq);
    const int warps = std::max(1, std::min(LRU_W, T / 8)), threads = 32 * warps;  // runs of at least 8 tokens; one warp when decoding
    if (out_f32)
        kf_rglru_scan_kernel<float><<<grid, threads, 0, ctx->stream>>>((float*)out, ldo, A, Bv, y_logit, ldy, (const uint16_t*)y_bias_bf16, state, state_stride, pos_dev,
                                                                 slot_dev, T, width);
    else
        kf_rglru_scan_kernel<uint16_t><<<grid, threads, 0, ctx->stream>>>((uint16_t*)out, ldo, A, Bv, y_logit, ldy, (const uint16_t*)y_bias_bf16, state, state_stride,
                                                                    pos_dev, slot_dev, T, width);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
