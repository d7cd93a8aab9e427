// attn_bias.cu -- causal grouped-query softmax attention whose score carries position terms instead of a rotation:
//     s_ij = (t_i q_i . k_j) * scale - r1_h * ln(1 + r2_h * (i - j)),   t_i = 1 + coef * ln(floor((i + 1) / every) + 1)
// (a logarithmic distance penalty per head and a query temperature that grows with the position), for any per-head key size dk and
// value size dv.  Cache rows hold [k (G x dk) | v (G x dv)] of one position in the activation type (bf16 bits or float); scores, the
// softmax and the weighted sum run in fp32.  One kernel serves prompts (M tokens of one slot) and decoding (one token of each of M
// slots): a CTA per (token, head), a lane per key for the scores (32 keys per warp step), lanes over the value entries for the sum,
// online softmax per warp, warps merged at the end.  The optional output gate sigmoid(g) is applied to the head's result before it
// is written in the activation type.  Beside kf_attn_* of attention.cu (rotated, head size 64 / 128, bf16 only, Qwen3's path).
#include <math.h>

#include <algorithm>

#include "kf_common.cuh"

namespace {
template <typename TC>
__device__ __forceinline__ float ldc(const TC* p);
template <>
__device__ __forceinline__ float ldc<uint16_t>(const uint16_t* p) { return bf16_bits_to_f32(*p); }
template <>
__device__ __forceinline__ float ldc<float>(const float* p) { return *p; }

template <typename TC>
__global__ void kf_kv_append_kernel(TC* __restrict__ cache, size_t slot_stride, int W, const float* __restrict__ k, int ldk, int nk, const float* __restrict__ v,
                                    int ldv, int nv, const int32_t* __restrict__ pos, const int32_t* __restrict__ slot) {
    const int m = blockIdx.x;
    TC* row = cache + (size_t)slot[m] * slot_stride + (size_t)pos[m] * W;
    for (int i = threadIdx.x; i < nk + nv; i += blockDim.x) {
        const float x = i < nk ? k[(size_t)m * ldk + i] : v[(size_t)m * ldv + i - nk];
        if (sizeof(TC) == 2) ((uint16_t*)row)[i] = f32_to_bf16_bits(x);
        else ((float*)row)[i] = x;
    }
}

// q_out[m][i] = bf16(q[m][i] * t(pos[m])): the query with its position's temperature, as the tensor-core panel kernel takes it
__global__ void kf_q_temp_kernel(uint16_t* __restrict__ q_out, const float* __restrict__ q, int ldq, const int32_t* __restrict__ pos, int n, float t_coef,
                                 int t_every) {
    const int m = blockIdx.x;
    const float temp = t_every > 0 ? 1.f + t_coef * logf((float)((pos[m] + 1) / t_every) + 1.f) : 1.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) q_out[(size_t)m * n + i] = f32_to_bf16_bits(q[(size_t)m * ldq + i] * temp);
}

struct AttnArgs {
    void* out;  // [M][ldo] activation type, heads x dv
    int ldo, out_f32;
    const float* q;  // [M][ldq] heads x dk
    int ldq;
    const float* gate;  // [M][ldg] heads x dv logits, or NULL
    int ldg;
    const void* cache;
    size_t slot_stride;
    const uint16_t *r1, *r2;  // bf16 [H] or NULL
    const int32_t *pos, *slot;
    int H, G, dk, dv;
    float scale, t_coef;
    int t_every;
    int nsplit;   // the keys of a token are dealt to nsplit CTAs (blockIdx.z); > 1: partial (max, sum, weighted values) go to ws
    float* ws;    // [M][H][nsplit][dv + 2]
};

constexpr int AW = 4;  // warps per CTA
template <typename TC, int VPL>
__global__ void __launch_bounds__(AW * 32) kf_attn_bias_kernel(AttnArgs a) {
    extern __shared__ float sm[];
    float* sq   = sm;                    // [dk]
    float* sacc = sq + a.dk;             // [AW][dv]
    float* sml  = sacc + AW * a.dv;      // [AW][2]
    const int m = blockIdx.x, h = blockIdx.y, kh = h / (a.H / a.G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = a.pos[m], W = a.G * (a.dk + a.dv);
    const TC* base = (const TC*)a.cache + (size_t)a.slot[m] * a.slot_stride;
    float temp = a.scale;
    if (a.t_every > 0) temp *= 1.f + a.t_coef * logf((float)((p + 1) / a.t_every) + 1.f);
    for (int d = threadIdx.x; d < a.dk; d += blockDim.x) sq[d] = a.q[(size_t)m * a.ldq + h * a.dk + d] * temp;
    __syncthreads();
    const float r1 = a.r1 ? bf16_bits_to_f32(a.r1[h]) : 0.f, r2 = a.r2 ? bf16_bits_to_f32(a.r2[h]) : 0.f;
    float mx = -INFINITY, l = 0.f, acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; i++) acc[i] = 0.f;
    const bool vec = sizeof(TC) == 2 && a.dk % 8 == 0 && W % 8 == 0 && (a.slot_stride % 8) == 0 && (((uintptr_t)a.cache & 15) == 0);
    // this CTA's keys: [j_lo, j_hi), whole 32-key steps per split
    const int chunk = a.nsplit > 1 ? (((p + a.nsplit) / a.nsplit + 31) & ~31) : p + 1;
    const int j_lo = blockIdx.z * chunk, j_hi = min(p + 1, j_lo + chunk);
    for (int j0 = j_lo + warp * 32; j0 < j_hi; j0 += AW * 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        if (j < j_hi) {
            const TC* kr = base + (size_t)j * W + kh * a.dk;
            float d0 = 0.f, d1 = 0.f;
            if (vec) {
                for (int d = 0; d < a.dk; d += 8) {
                    const uint4 kv = *reinterpret_cast<const uint4*>((const uint16_t*)kr + d);
                    d0 = fmaf(bf16lo(kv.x), sq[d], d0), d1 = fmaf(bf16hi(kv.x), sq[d + 1], d1);
                    d0 = fmaf(bf16lo(kv.y), sq[d + 2], d0), d1 = fmaf(bf16hi(kv.y), sq[d + 3], d1);
                    d0 = fmaf(bf16lo(kv.z), sq[d + 4], d0), d1 = fmaf(bf16hi(kv.z), sq[d + 5], d1);
                    d0 = fmaf(bf16lo(kv.w), sq[d + 6], d0), d1 = fmaf(bf16hi(kv.w), sq[d + 7], d1);
                }
            } else {
                for (int d = 0; d < a.dk; d++) d0 = fmaf(ldc<TC>(kr + d), sq[d], d0);
            }
            s = d0 + d1;
            if (a.r1) s -= r1 * log1pf(r2 * (float)(p - j));
        }
        const float bm = warp_max(s), nm = fmaxf(mx, bm);
        const float corr = expf(mx - nm), pj = j < j_hi ? expf(s - nm) : 0.f;  // mx = -inf on the first pass: corr = 0
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < VPL; i++) acc[i] *= corr;
        mx = nm;
        const int nk = min(32, j_hi - j0);
        // U keys per step: their value loads are issued together (a key past the range repeats the last row with weight 0)
        constexpr int U = VPL <= 4 ? 4 : (VPL <= 8 ? 2 : 1);
        for (int t = 0; t < nk; t += U) {
            float pt[U], x[U][VPL];
#pragma unroll
            for (int e = 0; e < U; e++) {
                pt[e] = __shfl_sync(0xffffffffu, pj, (t + e) & 31);
                const TC* vr = base + (size_t)min(j0 + t + e, j_hi - 1) * W + a.G * a.dk + kh * a.dv;
#pragma unroll
                for (int i = 0; i < VPL; i++) {
                    const int d = i * 32 + lane;
                    x[e][i] = d < a.dv ? ldc<TC>(vr + d) : 0.f;
                }
            }
#pragma unroll
            for (int e = 0; e < U; e++)
#pragma unroll
                for (int i = 0; i < VPL; i++) acc[i] = fmaf(pt[e], x[e][i], acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        const int d = i * 32 + lane;
        if (d < a.dv) sacc[warp * a.dv + d] = acc[i];
    }
    if (lane == 0) sml[warp * 2] = mx, sml[warp * 2 + 1] = l;
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < AW; w++) M = fmaxf(M, sml[w * 2]);
    float L = 0.f, f[AW];
    for (int w = 0; w < AW; w++) f[w] = sml[w * 2] == -INFINITY ? 0.f : expf(sml[w * 2] - M), L += f[w] * sml[w * 2 + 1];
    if (a.nsplit > 1) {  // partial result of this split; kf_attn_bias_merge_kernel finishes
        float* part = a.ws + (((size_t)m * a.H + h) * a.nsplit + blockIdx.z) * (a.dv + 2);
        if (threadIdx.x == 0) part[0] = M, part[1] = L;
        for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
            float o = 0.f;
            for (int w = 0; w < AW; w++) o = fmaf(f[w], sacc[w * a.dv + d], o);
            part[2 + d] = o;
        }
        return;
    }
    for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < AW; w++) o = fmaf(f[w], sacc[w * a.dv + d], o);
        o /= L;
        if (a.gate) {
            const float z = a.gate[(size_t)m * a.ldg + h * a.dv + d];
            o *= 1.f / (1.f + expf(-z));
        }
        if (a.out_f32) ((float*)a.out)[(size_t)m * a.ldo + h * a.dv + d] = o;
        else ((uint16_t*)a.out)[(size_t)m * a.ldo + h * a.dv + d] = f32_to_bf16_bits(o);
    }
}
// the splits of one (token, head) merged in split order, gated, written in the activation type
__global__ void kf_attn_bias_merge_kernel(AttnArgs a) {
    const int m = blockIdx.x, h = blockIdx.y;
    const float* part = a.ws + ((size_t)m * a.H + h) * a.nsplit * (a.dv + 2);
    float M = -INFINITY;
    for (int z = 0; z < a.nsplit; z++) M = fmaxf(M, part[(size_t)z * (a.dv + 2)]);
    float L = 0.f;
    for (int z = 0; z < a.nsplit; z++) {
        const float mz = part[(size_t)z * (a.dv + 2)];
        if (mz != -INFINITY) L += expf(mz - M) * part[(size_t)z * (a.dv + 2) + 1];
    }
    for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < a.nsplit; z++) {
            const float mz = part[(size_t)z * (a.dv + 2)];
            if (mz != -INFINITY) o = fmaf(expf(mz - M), part[(size_t)z * (a.dv + 2) + 2 + d], o);
        }
        o /= L;
        if (a.gate) {
            const float z = a.gate[(size_t)m * a.ldg + h * a.dv + d];
            o *= 1.f / (1.f + expf(-z));
        }
        if (a.out_f32) ((float*)a.out)[(size_t)m * a.ldo + h * a.dv + d] = o;
        else ((uint16_t*)a.out)[(size_t)m * a.ldo + h * a.dv + d] = f32_to_bf16_bits(o);
    }
}
}  // namespace

// cache[slot[m]][pos[m]] = [k row (nk floats) | v row (nv floats)] in the cache's type
extern "C" int kf_kv_append(kf_ctx* ctx, void* cache, int cache_f32, size_t slot_stride, const float* k, int ldk, int nk, const float* v, int ldv, int nv,
                            const int32_t* pos_dev, const int32_t* slot_dev, int M) {
    if (!ctx || !cache || !k || !v || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, M >= 1 && nk >= 1 && nv >= 1, "shape");
    if (cache_f32) kf_kv_append_kernel<float><<<M, 256, 0, ctx->stream>>>((float*)cache, slot_stride, nk + nv, k, ldk, nk, v, ldv, nv, pos_dev, slot_dev);
    else kf_kv_append_kernel<uint16_t><<<M, 256, 0, ctx->stream>>>((uint16_t*)cache, slot_stride, nk + nv, k, ldk, nk, v, ldv, nv, pos_dev, slot_dev);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
// out [M][ldo] (heads x dv, activation type) = attention of token m over the rows 0 .. pos[m] of its slot (its own row appended before).
// r1 / r2: bf16 [H] distance-penalty numbers or NULL; t_every <= 0: no query temperature; gate_logit: float [M][ldg] or NULL;
// max_pos_hint: an upper bound of pos[] (sizes the split of the keys over CTAs; the result does not depend on it beyond rounding).
extern "C" int kf_attn_bias(kf_ctx* ctx, void* out, int out_f32, int ldo, const float* q, int ldq, const float* gate_logit, int ldg, const void* cache,
                            int cache_f32, size_t slot_stride, const void* r1_bf16, const void* r2_bf16, const int32_t* pos_dev, const int32_t* slot_dev,
                            int M, int H, int G, int dk, int dv, float scale, float t_coef, int t_every, int max_pos_hint) {
    if (!ctx || !out || !q || !cache || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, M >= 1 && H >= 1 && G >= 1 && H % G == 0 && dk >= 1 && dv >= 1 && dv <= 512 && (!r1_bf16) == (!r2_bf16), "value size <= 512, kv heads divide heads");
    AttnArgs a = {};
    a.out = out, a.ldo = ldo, a.out_f32 = out_f32, a.q = q, a.ldq = ldq, a.gate = gate_logit, a.ldg = ldg, a.cache = cache, a.slot_stride = slot_stride;
    a.r1 = (const uint16_t*)r1_bf16, a.r2 = (const uint16_t*)r2_bf16, a.pos = pos_dev, a.slot = slot_dev, a.H = H, a.G = G, a.dk = dk, a.dv = dv;
    a.scale = scale, a.t_coef = t_coef, a.t_every = t_every;
    const size_t smem = (size_t)(dk + AW * dv + AW * 2) * sizeof(float);
    KF_REQUIRE(ctx, smem <= 48 * 1024, "key size");
    // few (token, head) pairs and long contexts (decoding): the keys are dealt to several CTAs so that the SMs are busy
    int nsplit = 1;
    if (M * H < 2 * ctx->sm_count && max_pos_hint >= 4 * AW * 32)
        nsplit = std::max(1, std::min(std::min(64, (2 * ctx->sm_count) / (M * H)), (max_pos_hint + 1) / (2 * AW * 32)));
    if (nsplit > 1) {
        KF_REQUIRE(ctx, kf_ensure_attn_ws(ctx, (size_t)M * H * nsplit * (dv + 2) * sizeof(float)) == KF_OK, "attention workspace");
        a.ws = ctx->attn_ws;
    }
    a.nsplit = nsplit;
    dim3 grid(M, H, nsplit);
    const int vpl = (dv + 31) / 32;
#define KF_AB(TC, V) kf_attn_bias_kernel<TC, V><<<grid, AW * 32, smem, ctx->stream>>>(a)
    if (cache_f32) {
        if (vpl <= 2) KF_AB(float, 2);
        else if (vpl <= 4) KF_AB(float, 4);
        else if (vpl <= 8) KF_AB(float, 8);
        else KF_AB(float, 16);
    } else {
        if (vpl <= 2) KF_AB(uint16_t, 2);
        else if (vpl <= 4) KF_AB(uint16_t, 4);
        else if (vpl <= 8) KF_AB(uint16_t, 8);
        else KF_AB(uint16_t, 16);
    }
#undef KF_AB
    KF_LAUNCH_CHECK(ctx);
    if (nsplit > 1) {
        kf_attn_bias_merge_kernel<<<dim3(M, H), 128, 0, ctx->stream>>>(a);
        KF_LAUNCH_CHECK(ctx);
    }
    return KF_OK;
}

// A panel of M consecutive tokens of ONE slot on the tensor cores (kf_attn_bias_prefill of attention.cu): bf16 cache, dk == dv in {64, 128}.
// q_work: bf16 scratch [M][H * hd].  Same result as kf_attn_bias up to the bf16 rounding of the tempered query.
extern "C" int kf_attn_bias_panel(kf_ctx* ctx, void* out_bf16, void* q_work_bf16, const float* q, int ldq, const float* gate_logit, int ldg, const void* cache,
                                  size_t slot_stride, const void* r1_bf16, const void* r2_bf16, const int32_t* pos_dev, const int32_t* slot_dev, int M, int H,
                                  int G, int hd, int max_seq, float scale, float t_coef, int t_every) {
    if (!ctx || !out_bf16 || !q_work_bf16 || !q) return KF_ERR_BAD_ARG;
    kf_q_temp_kernel<<<M, 256, 0, ctx->stream>>>((uint16_t*)q_work_bf16, q, ldq, pos_dev, H * hd, t_coef, t_every);
    KF_LAUNCH_CHECK(ctx);
    return kf_attn_bias_prefill(ctx, out_bf16, q_work_bf16, cache, slot_stride, r1_bf16, r2_bf16, gate_logit, ldg, pos_dev, slot_dev, M, H, G, hd, max_seq, scale);
}
