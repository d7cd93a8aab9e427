// Kivorax.hpp -- neurons of the Kivorax stack.  Every layer normalises once and both of its sublayers work from that copy, their
// results going into the residual together (x += mixer(norm(x)) + ff(norm(x))); then comes a per-layer token input (a slice of a second
// embedding gates a small projection of x, RMS-normed and added), then the depth average: the next layer does not read this layer's
// result but a learned weighted sum of the embedding output and of all layer results so far.  Mixers: the gated delta rule and
// gated linear attention (matrix-state recurrences, DeltaMixer / GLAMixer), and attention with a distance penalty beside a real-gated
// linear recurrent unit (PairMixer).  Feed-forward: dense with biases, or routed experts weighted by the full softmax.  The residual,
// norms, router, recurrences and attention scores are fp32; matmul inputs are written in the activation type.  The neurons use the
// model's HybridScratch and SeqStateCache (Sipazen.hpp, QWen3.hpp); step function, graphs, sampler and generation loop are Fish's own.
// The reference has no counterpart (its inference path is the Qwen3 block, QWen.cpp:16-145).
#pragma once
#include "Sipazen.hpp"

namespace koifish {

struct DeltaMixer : GeNeuron {  // gated delta rule with short convolutions on q, k, v
    MIXER_CARD card;
    int layer = 0;
    hGTensor q, k, v, qc, kc, vc, b, A_log, norm, a1, a2, dt_bias, g1, g2, o;
    StackedLinear convs;  // q.conv | k.conv | v.conv as one [channels][taps] table
    int cuInfer(int M, const float* u, int ldu, const int* off);  // off: columns of q, b, a1 in the stacked projections
};
struct GLAMixer : GeNeuron {  // gated linear attention
    MIXER_CARD card;
    int layer = 0;
    hGTensor q, k, v, g, o, norm, a1, a2, a2_b;
    int cuInfer(int M, const float* u, int ldu, const int* off);  // off: q, k, v, g, a1
};
struct PairMixer : GeNeuron {  // attention (left) beside a real-gated LRU (right), each RMS-normed, half the sum
    MIXER_CARD card;
    int layer = 0;
    hGTensor lq, lk, lv, lg, lo, r1, r2, lout;
    hGTensor ry, ry_b, rx, rx_b, conv, conv_b, ra, ra_b, ri, ri_b, lam, ro, rout;
    int cuInfer(int M, float* u, int ldu, const int* off);  // off: q, k, v, g, y, x ; adds to the residual itself
};
struct KvxFF : GeNeuron {  // dense (up, gelu, down, biases) or routed experts (relu squared, full-softmax weights)
    MOE_CARD card;
    hGTensor up, up_b, down, down_b, router;
    std::vector<hGTensor> eup, edown;
    void** tables = nullptr;  // device [2][experts]: up | down
    int Prepare();
    int cuInfer(int M, const float* u, int ldu, int off);  // adds to the residual
};
struct KvxBlock : GeNeuron {
    int layer = 0;
    GroupNorm norm1;
    StackedLinear cat;  // everything that reads h: the mixer's first projections, then the dense up projection or the router
    std::vector<int> off;
    std::unique_ptr<DeltaMixer> delta;
    std::unique_ptr<GLAMixer> gla;
    std::unique_ptr<PairMixer> pair;
    std::unique_ptr<KvxFF> ff;
    hGTensor side_gate, side_proj, side_norm, dwa;
    int cuInfer(int M);
};

}  // namespace koifish
