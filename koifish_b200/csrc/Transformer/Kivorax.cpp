// Kivorax.cpp -- config parsing, construction and the per-layer step of the Kivorax stack (see Kivorax.hpp).
#include "Kivorax.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>

namespace koifish {

#define KF_TRY(expr)                                                                       \
    do {                                                                                   \
        int _rc = (expr);                                                                  \
        if (_rc != KF_OK) {                                                                \
            *hFishErr = std::string(#expr) + " -> " + kf_status_string(_rc);               \
            return _rc;                                                                    \
        }                                                                                  \
    } while (0)

// ------------------------------------------------------------------------------------------------------------ config
static int need_int(const JSON& j, const char* key, const std::string& where) {
    const JSON* p = j.find(key);
    if (!p || !p->is_number()) throw std::runtime_error("config: " + where + "." + key + " is missing");
    return p->as_int();
}
// A size that the config does not carry: the mixer's own key when present, else the first extent of the named tensor in "tensor_shapes"
// (the loader puts the checkpoint's shapes there).
static int shape_int(const JSON& h, const JSON& mixer, const char* key, const std::string& tensor, const std::string& where) {
    if (mixer.contains(key)) return need_int(mixer, key, where);
    if (const JSON* ts = h.find("tensor_shapes"))
        if (const JSON* t = ts->find(tensor))
            if (t->is_array() && !t->arr.empty()) return t->arr[0].as_int();
    throw std::runtime_error("config: " + where + "." + key + " is neither in the config nor given by the shape of '" + tensor + "'");
}
// config.json: {"architecture": "Kivorax", "vocab", "width", "embedding": {"scale"}, "norm": {"eps"}, "token_side": {"dim"},
//               "layers": [{"type": "channel_delta" | "gla" | "parallel", "mixer": {...}, "mlp": {"kind": "dense" | "moe", ...} | null}]}
static void ParseKivorax(const JSON& h, MODEL_CARD& c) {
    c.vocab  = need_int(h, "vocab", "config");
    c.n_embd = need_int(h, "width", "config");
    if (const JSON* e = h.find("embedding"))
        if (const JSON* s = e->find("scale")) c.embed_scale = (float)s->as_double(1.0);
    c.norm_rms_eps = (float)h.at("norm").at("eps").as_double(1e-5);
    c.norm_groups  = 1;
    if (const JSON* t = h.find("token_side"))
        if (!t->is_null()) c.side_dim = need_int(*t, "dim", "token_side");
    const JSON& ls = h.at("layers");
    if (!ls.is_array() || ls.arr.empty()) throw std::runtime_error("config: layers must be a non-empty list");
    for (size_t i = 0; i < ls.arr.size(); i++) {
        const JSON& l = ls.arr[i];
        const std::string where = "layers[" + std::to_string(i) + "]", tp = "l" + std::to_string(i) + ".mix.";
        LAYER_CARD lc;
        MIXER_CARD& m = lc.mixer;
        m.type        = l.at("type").as_string();
        const JSON& x = l.at("mixer");
        if (m.type == "channel_delta") {
            m.heads = need_int(x, "heads", where), m.kv_heads = x.contains("kv_heads") ? need_int(x, "kv_heads", where) : m.heads;
            m.dim = need_int(x, "dim", where), m.vdim = need_int(x, "vdim", where), m.conv = need_int(x, "conv", where);
            m.rank_a = shape_int(h, x, "a_rank", tp + "a1", where), m.rank_g = shape_int(h, x, "g_rank", tp + "g1", where);
            if (m.heads < 1 || m.kv_heads < 1 || m.heads % m.kv_heads || m.dim < 1 || m.dim > 512 || m.vdim < 1 || m.conv < 1 || m.rank_a < 1 || m.rank_g < 1)
                throw std::runtime_error("config: " + where + ": kv_heads must divide heads; 1 <= dim <= 512");
        } else if (m.type == "gla") {
            m.heads = m.kv_heads = need_int(x, "heads", where), m.dim = need_int(x, "dim", where), m.vdim = need_int(x, "vdim", where);
            m.tau    = (float)x.at("tau").as_double(1.0);
            m.rank_a = shape_int(h, x, "a_rank", tp + "a1", where);
            if (m.heads < 1 || m.dim < 1 || m.dim > 512 || m.vdim < 1 || !(m.tau > 0.f) || m.rank_a < 1)
                throw std::runtime_error("config: " + where + ": 1 <= dim <= 512, tau > 0");
        } else if (m.type == "parallel") {
            const JSON& a = x.at("left");
            const JSON& r = x.at("right");
            m.heads = need_int(a, "heads", where), m.kv_heads = a.contains("kv_heads") ? need_int(a, "kv_heads", where) : m.heads;
            m.dim = need_int(a, "dim", where), m.vdim = need_int(a, "vdim", where);
            m.scale = a.contains("scale") ? (float)a.at("scale").as_double(1.0) : 1.0f / std::sqrt((float)m.dim);
            if (const JSON* t = a.find("q_temp"))
                if (!t->is_null()) m.qt_coef = (float)t->at("coef").as_double(0.0), m.qt_every = need_int(*t, "every", where + ".q_temp");
            m.lru_width = need_int(r, "width", where), m.lru_blocks = need_int(r, "blocks", where), m.lru_conv = need_int(r, "conv", where);
            if (m.heads < 1 || m.kv_heads < 1 || m.heads % m.kv_heads || m.dim < 1 || m.vdim < 1 || m.vdim > 512 || m.qt_every < 0 || m.lru_width < 1 ||
                m.lru_blocks < 1 || m.lru_width % m.lru_blocks || m.lru_conv < 1)
                throw std::runtime_error("config: " + where + ": kv_heads must divide heads, blocks must divide width, vdim <= 512");
        } else {
            throw std::runtime_error("config: " + where + ": unknown mixer type '" + m.type + "'");
        }
        const JSON* f = l.find("mlp");
        if (f && !f->is_null()) {
            const std::string kind = f->at("kind").as_string();
            lc.mlp.present = true;
            if (kind == "dense") {
                lc.mlp.dense = true, lc.mlp.ff = need_int(*f, "ff", where + ".mlp");
            } else if (kind == "moe") {
                lc.mlp.experts = need_int(f->at("router"), "experts", where + ".mlp.router");
                lc.mlp.top     = need_int(f->at("router"), "top", where + ".mlp.router");
                lc.mlp.ff      = need_int(f->at("expert"), "ff", where + ".mlp.expert");
                if (lc.mlp.experts < 1 || lc.mlp.top < 1 || lc.mlp.top > lc.mlp.experts) throw std::runtime_error("config: " + where + ".mlp: 1 <= top <= experts");
            } else {
                throw std::runtime_error("config: " + where + ".mlp.kind '" + kind + "' is not built");
            }
            if (lc.mlp.ff < 1) throw std::runtime_error("config: " + where + ".mlp: ff must be positive");
        }
        c.layers.push_back(lc);
    }
    c.n_layers = (int)c.layers.size();
    if (c.vocab < 1 || c.n_embd < 1 || c.side_dim < 0) throw std::runtime_error("config: vocab, width must be positive");
    c.n_head = c.n_head_kv = 1, c.head_dim = c.n_embd, c.n_ff = 0, c.tie_word_embeddings = false;
}

// ------------------------------------------------------------------------------------------------------------ build
namespace {
struct Builder {
    Fish& f;
    int next_id = 0;
    void Tensor(const std::string& name, int rows, int cols, hGTensor& out) {
        out = std::make_shared<GTensor>(f.ctx, name, rows, cols);  // bf16 as stored
        f.tensors[name]    = out;
        f.tensor_ids[name] = next_id++;
    }
    template <typename T>
    int Buf(T** p, size_t bytes) {
        void* d = nullptr;
        int rc  = kf_malloc(f.ctx, std::max<size_t>(bytes, 16), &d);
        if (rc) return rc;
        f.owned.push_back(d);
        *p = (T*)d;
        return KF_OK;
    }
};
}  // namespace

static int BuildKivorax(Fish& f) {
    std::string* hFishErr = &f.error;
    const MODEL_CARD& c   = f.config;
    if (f.tp_world != 1) {
        f.error = "the Kivorax stack runs on one GPU (no tensor-parallel shard plan)";
        return KF_ERR_UNSUPPORTED;
    }
    Builder b{f};
    const int E = c.n_embd, L = (int)c.layers.size();
    const bool f32   = c.compute_f32;
    const size_t asz = f32 ? 4 : 2;
    f.embed.hFish = &f, f.embed.name = "embed";
    b.Tensor("embed", c.vocab, E, f.embed.w);
    hGTensor side_embed;
    if (c.side_dim > 0) b.Tensor("side.embed", c.vocab, L * c.side_dim, side_embed);
    f.cls.hFish = &f, f.cls.name = "head";
    f.cls.norm.hFish = &f, f.cls.norm.rms_eps = c.norm_rms_eps;
    b.Tensor("final.norm", 1, E, f.cls.norm.w);
    f.cls.proj.hFish = &f, f.cls.proj.nIn = E, f.cls.proj.nOut = c.vocab;
    b.Tensor("head", c.vocab, E, f.cls.proj.w);

    f.max_tokens = std::max(std::max(64, c.max_batch), c.max_prefill);
    f.logit_rows = c.logit_rows_cfg > 0 ? std::min(c.logit_rows_cfg, f.max_tokens) : std::max(64, c.max_batch);
    const size_t T = f.max_tokens;
    auto hs    = std::make_shared<HybridScratch>();
    f.hscratch = hs;
    size_t maxU = 1, maxV = std::max(1, c.side_dim), maxY = 1, maxL = 1, maxA = 1, maxMid = std::max(1, c.side_dim), maxE = 1, maxSlots = 1, maxH1 = 1, maxW = 1;
    f.states.layers.resize(L);
    f.states.max_seq = c.max_seq_len, f.states.f32 = f32;
    for (int i = 0; i < L; i++) {
        const LAYER_CARD& lc = c.layers[i];
        const MIXER_CARD& m  = lc.mixer;
        const std::string p = "l" + std::to_string(i) + ".", mp = p + "mix.";
        auto blk   = std::make_unique<KvxBlock>();
        blk->hFish = &f, blk->name = p, blk->layer = i;
        blk->norm1.hFish = &f, blk->norm1.groups = 1, blk->norm1.eps = c.norm_rms_eps;
        b.Tensor(p + "norm1", 1, E, blk->norm1.w);
        SeqStateCache::Layer& sl = f.states.layers[i];
        std::vector<hGTensor> parts;
        if (m.type == "channel_delta") {
            auto d = std::make_unique<DeltaMixer>();
            d->hFish = &f, d->name = mp, d->card = m, d->layer = i;
            const int nq = m.kv_heads * m.dim, nv = m.heads * m.vdim, C = 2 * nq + nv;
            b.Tensor(mp + "q", nq, E, d->q), b.Tensor(mp + "q.conv", nq, m.conv, d->qc);
            b.Tensor(mp + "k", nq, E, d->k), b.Tensor(mp + "k.conv", nq, m.conv, d->kc);
            b.Tensor(mp + "v", nv, E, d->v), b.Tensor(mp + "v.conv", nv, m.conv, d->vc);
            b.Tensor(mp + "b", m.heads, E, d->b);
            b.Tensor(mp + "A_log", 1, m.heads, d->A_log);
            b.Tensor(mp + "norm", 1, m.vdim, d->norm);
            b.Tensor(mp + "a1", m.rank_a, E, d->a1), b.Tensor(mp + "a2", m.heads * m.dim, m.rank_a, d->a2);
            b.Tensor(mp + "dt_bias", 1, m.heads * m.dim, d->dt_bias);
            b.Tensor(mp + "g1", m.rank_g, E, d->g1), b.Tensor(mp + "g2", nv, m.rank_g, d->g2);
            b.Tensor(mp + "o", E, nv, d->o);
            d->convs.Plan({d->qc, d->kc, d->vc});
            KF_TRY(b.Buf((char**)&d->convs.w, (size_t)d->convs.rows * m.conv * 2));
            sl.state_stride = (size_t)m.heads * m.dim * m.vdim;
            sl.tail_stride  = (size_t)std::max(1, m.conv - 1) * C;
            parts = {d->q, d->k, d->v, d->b, d->a1, d->g1};
            maxV = std::max<size_t>(maxV, C), maxY = std::max<size_t>(maxY, nv), maxA = std::max<size_t>(maxA, nv);
            maxL = std::max<size_t>(maxL, (size_t)m.heads * m.dim + nv), maxMid = std::max<size_t>(maxMid, m.rank_a + m.rank_g);
            blk->delta = std::move(d);
        } else if (m.type == "gla") {
            auto g = std::make_unique<GLAMixer>();
            g->hFish = &f, g->name = mp, g->card = m, g->layer = i;
            const int nq = m.heads * m.dim, nv = m.heads * m.vdim;
            b.Tensor(mp + "q", nq, E, g->q), b.Tensor(mp + "k", nq, E, g->k), b.Tensor(mp + "v", nv, E, g->v), b.Tensor(mp + "g", nv, E, g->g);
            b.Tensor(mp + "o", E, nv, g->o);
            b.Tensor(mp + "norm", 1, m.vdim, g->norm);
            b.Tensor(mp + "a1", m.rank_a, E, g->a1), b.Tensor(mp + "a2", nq, m.rank_a, g->a2), b.Tensor(mp + "a2.b", 1, nq, g->a2_b);
            sl.state_stride = (size_t)m.heads * m.dim * m.vdim;
            parts = {g->q, g->k, g->v, g->g, g->a1};
            maxY = std::max<size_t>(maxY, nv), maxA = std::max<size_t>(maxA, nv), maxL = std::max<size_t>(maxL, nq), maxMid = std::max<size_t>(maxMid, m.rank_a);
            blk->gla = std::move(g);
        } else {
            auto a = std::make_unique<PairMixer>();
            a->hFish = &f, a->name = mp, a->card = m, a->layer = i;
            const std::string lp = mp + "left.", rp = mp + "right.";
            const int nq = m.heads * m.dim, nk = m.kv_heads * m.dim, nv = m.kv_heads * m.vdim, no = m.heads * m.vdim, Wd = m.lru_width, bs = Wd / m.lru_blocks;
            b.Tensor(lp + "q", nq, E, a->lq), b.Tensor(lp + "k", nk, E, a->lk), b.Tensor(lp + "v", nv, E, a->lv), b.Tensor(lp + "g", no, E, a->lg);
            b.Tensor(lp + "r1", 1, m.heads, a->r1), b.Tensor(lp + "r2", 1, m.heads, a->r2);
            b.Tensor(lp + "o", E, no, a->lo), b.Tensor(lp + "out", 1, E, a->lout);
            b.Tensor(rp + "y", Wd, E, a->ry), b.Tensor(rp + "y.b", 1, Wd, a->ry_b), b.Tensor(rp + "x", Wd, E, a->rx), b.Tensor(rp + "x.b", 1, Wd, a->rx_b);
            b.Tensor(rp + "conv", Wd, m.lru_conv, a->conv), b.Tensor(rp + "conv.b", 1, Wd, a->conv_b);
            b.Tensor(rp + "ra", m.lru_blocks * bs, bs, a->ra), b.Tensor(rp + "ra.b", m.lru_blocks, bs, a->ra_b);
            b.Tensor(rp + "ri", m.lru_blocks * bs, bs, a->ri), b.Tensor(rp + "ri.b", m.lru_blocks, bs, a->ri_b);
            b.Tensor(rp + "lam", 1, Wd, a->lam);
            b.Tensor(rp + "o", E, Wd, a->ro), b.Tensor(rp + "out", 1, E, a->rout);
            sl.row_dim = nk + nv, sl.row_stride = (size_t)c.max_seq_len * sl.row_dim;
            sl.state_stride = Wd, sl.tail_stride = (size_t)std::max(1, m.lru_conv - 1) * Wd;
            parts = {a->lq, a->lk, a->lv, a->lg, a->ry, a->rx};
            maxV = std::max<size_t>(maxV, Wd), maxA = std::max<size_t>(maxA, std::max(no, Wd)), maxW = std::max<size_t>(maxW, Wd);
            maxY = std::max<size_t>(maxY, nq);  // the tempered bf16 query of the panel kernel
            blk->pair = std::move(a);
        }
        if (sl.row_stride) {  // zeroed once: the panel kernel may load rows beyond the sequence's end (masked, but they must hold numbers)
            KF_TRY(b.Buf((char**)&sl.rows, (size_t)c.max_batch * sl.row_stride * asz));
            KF_TRY(kf_memset(f.ctx, sl.rows, 0, (size_t)c.max_batch * sl.row_stride * asz));
        }
        if (sl.state_stride) KF_TRY(b.Buf(&sl.state, (size_t)c.max_batch * sl.state_stride * 4));
        if (sl.tail_stride) KF_TRY(b.Buf(&sl.tail, (size_t)c.max_batch * sl.tail_stride * 4));
        f.states.total_bytes += (size_t)c.max_batch * (sl.row_stride * asz + (sl.state_stride + sl.tail_stride) * 4);
        if (lc.mlp.present) {
            const MOE_CARD& mc = lc.mlp;
            auto e = std::make_unique<KvxFF>();
            e->hFish = &f, e->name = p + "mlp", e->card = mc;
            if (mc.dense) {
                b.Tensor(p + "mlp.up", mc.ff, E, e->up), b.Tensor(p + "mlp.up.b", 1, mc.ff, e->up_b);
                b.Tensor(p + "mlp.down", E, mc.ff, e->down), b.Tensor(p + "mlp.down.b", 1, E, e->down_b);
                parts.push_back(e->up);
                maxH1 = std::max<size_t>(maxH1, mc.ff);
            } else {
                e->eup.resize(mc.experts), e->edown.resize(mc.experts);
                for (int k = 0; k < mc.experts; k++) {
                    const std::string ep = p + "mlp.e" + std::to_string(k) + ".";
                    b.Tensor(ep + "up", mc.ff, E, e->eup[k]), b.Tensor(ep + "down", E, mc.ff, e->edown[k]);
                }
                b.Tensor(p + "mlp.router", mc.experts, E, e->router);
                KF_TRY(b.Buf(&e->tables, (size_t)2 * mc.experts * sizeof(void*)));
                parts.push_back(e->router);
                maxE = std::max<size_t>(maxE, mc.experts), maxSlots = std::max<size_t>(maxSlots, mc.top);
                maxH1 = std::max<size_t>(maxH1, (size_t)mc.top * mc.ff);
            }
            blk->ff = std::move(e);
        }
        b.Tensor(p + "dwa", 1, i + 2, blk->dwa);
        if (c.side_dim > 0) {
            b.Tensor(p + "side.gate", c.side_dim, E, blk->side_gate), b.Tensor(p + "side.proj", E, c.side_dim, blk->side_proj);
            b.Tensor(p + "side.norm", 1, E, blk->side_norm);
        }
        blk->cat.Plan(parts);
        blk->off = blk->cat.off;
        KF_TRY(b.Buf((char**)&blk->cat.w, (size_t)blk->cat.rows * E * 2));
        KF_TRY(kf_memset(f.ctx, blk->cat.w, 0, (size_t)blk->cat.rows * E * 2));
        maxU = std::max<size_t>(maxU, blk->cat.rows);
        f.blocks.push_back(std::move(blk));
    }
    // activations: fp32 residual stream and layer history; matmul inputs in the activation type
    KF_TRY(kf_malloc(f.ctx, T * E * 4, &f.x));
    KF_TRY(b.Buf(&hs->hist, (size_t)(L + 1) * T * E * 4));
    KF_TRY(b.Buf((char**)&hs->hact, T * E * asz));
    KF_TRY(b.Buf(&hs->sub, T * E * 4));
    KF_TRY(b.Buf(&hs->u, T * maxU * 4));
    KF_TRY(b.Buf(&hs->v, T * maxV * 4));
    KF_TRY(b.Buf(&hs->y, T * maxY * 4));
    KF_TRY(b.Buf(&hs->lat, T * maxL * 4));
    KF_TRY(b.Buf((char**)&hs->act, T * maxA * asz));
    KF_TRY(b.Buf((char**)&hs->mid, T * maxMid * asz));
    KF_TRY(b.Buf(&hs->lru_work, 2 * T * maxW * 4));
    const size_t TT = T * maxSlots;
    KF_TRY(b.Buf(&hs->idx, TT * 4));
    KF_TRY(b.Buf(&hs->wgt, TT * 4));
    KF_TRY(b.Buf(&hs->offsets, (maxE + 1) * 4));
    KF_TRY(b.Buf(&hs->entry_slot, TT * 4));
    KF_TRY(b.Buf(&hs->slot_row, TT * 4));
    KF_TRY(b.Buf(&hs->slot_group, TT * 4));
    KF_TRY(b.Buf(&hs->work, (2 * TT + maxE) * 4));
    KF_TRY(b.Buf((char**)&hs->h1, T * maxH1 * asz));
    KF_TRY(b.Buf(&hs->yslots, TT * E * 4));
    KF_TRY(b.Buf((char**)&hs->head_in, (size_t)f.logit_rows * E * asz));
    KF_TRY(kf_malloc(f.ctx, (size_t)f.logit_rows * c.vocab * 2, &f.logits));
    KF_TRY(kf_malloc(f.ctx, (size_t)f.logit_rows * c.vocab * 4, (void**)&f.logits_f32));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_tokens));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_pos));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_next));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_slot));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_sel));
    KF_TRY(kf_host_alloc(T * 4 * 5, (void**)&f.h_stage));
    KF_TRY(kf_host_alloc((size_t)f.logit_rows * c.vocab * 2, (void**)&f.h_logits));
    KF_TRY(kf_host_alloc((size_t)f.logit_rows * c.vocab * 4, (void**)&f.h_logits_f32));
    f.attn_hint = c.max_seq_len - 1;
    return KF_OK;
}

int KvxFF::Prepare() {
    if (card.dense) return KF_OK;
    Fish& f = *hFish;
    std::vector<const void*> t((size_t)2 * card.experts);
    for (int k = 0; k < card.experts; k++) t[k] = eup[k]->data, t[card.experts + k] = edown[k]->data;
    int rc = kf_h2d(f.ctx, tables, t.data(), t.size() * sizeof(void*));
    if (!rc) rc = kf_ctx_sync(f.ctx);
    return rc;
}
static int PrepareKivorax(Fish& f) {
    for (auto& n : f.blocks) {
        KvxBlock* b = static_cast<KvxBlock*>(n.get());
        int rc = b->cat.Fill(f.ctx);
        if (!rc && b->delta) rc = b->delta->convs.Fill(f.ctx);
        if (!rc && b->ff) rc = b->ff->Prepare();
        if (rc) return rc;
    }
    return KF_OK;
}

// ------------------------------------------------------------------------------------------------------------ step
static int Lin(Fish& f, float* y, int ldy, const hGTensor& w, const void* x, int ldx, int M) {
    kf_tensor_desc d = w->Desc();
    return kf_linear_g(f.ctx, y, ldy, &d, x, f.config.compute_f32 ? 1 : 0, ldx, M);
}
// x += v (+ bias)
static int AddTo(Fish& f, const float* v, const hGTensor& bias, int M) {
    const int E = f.config.n_embd;
    return kf_bias_act(f.ctx, f.x, 2, E, v, E, bias ? bias->data : nullptr, 0, nullptr, 0, M, E);
}

int DeltaMixer::cuInfer(int M, const float* u, int ldu, const int* off) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MIXER_CARD& m = card;
    const int ak = f.config.compute_f32 ? 1 : 0;
    const size_t asz = ak ? 4 : 2;
    const int nq = m.kv_heads * m.dim, nv = m.heads * m.vdim, C = 2 * nq + nv, nz = m.heads * m.dim, Lw = nz + nv, R = m.rank_a + m.rank_g;
    const int nseq = f.seq_mode ? M : 1, T = f.seq_mode ? 1 : M;
    SeqStateCache::Layer& sl = f.states.layers[layer];
    // q | k | v through their short convolutions and SiLU (one launch: the three tables are stacked like the projections)
    KF_TRY(kf_conv1d(f.ctx, s.v, u, ldu, off[0], convs.w, nullptr, sl.tail, sl.tail_stride, f.d_pos, f.d_slot, nseq, T, C, m.conv, 1));
    // second stage of the low-rank decay and gate projections
    KF_TRY(kf_bias_act(f.ctx, s.mid, ak ? 1 : 0, R, u + off[4], ldu, nullptr, 0, nullptr, 0, M, R));
    KF_TRY(Lin(f, s.lat, Lw, a2, s.mid, R, M));
    KF_TRY(Lin(f, s.lat + nz, Lw, g2, (const char*)s.mid + (size_t)m.rank_a * asz, R, M));
    KF_TRY(kf_gated_scan(f.ctx, s.y, nv, s.v, C, s.v + nq, C, s.v + 2 * nq, C, s.lat, Lw, dt_bias->data, A_log->data, u + off[3], ldu, sl.state, sl.state_stride,
                         f.d_pos, f.d_slot, nseq, T, m.heads, m.kv_heads, m.dim, m.vdim, 1, 1, 1.f, 1, 1e-6f, 1.0f / std::sqrt((float)m.dim)));
    // per-head RMS norm (weight shared by the heads) times sigmoid(gate)
    KF_TRY(kf_group_rmsnorm_ex(f.ctx, s.act, ak, nv, nullptr, 0.f, s.y, nv, s.lat + nz, Lw, nullptr, 3, norm->data, 1, nullptr, M, nv, m.heads,
                               f.config.norm_rms_eps));
    KF_TRY(Lin(f, s.sub, f.config.n_embd, o, s.act, nv, M));
    return AddTo(f, s.sub, nullptr, M);
}

int GLAMixer::cuInfer(int M, const float* u, int ldu, const int* off) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MIXER_CARD& m = card;
    const int ak = f.config.compute_f32 ? 1 : 0;
    const int nq = m.heads * m.dim, nv = m.heads * m.vdim;
    const int nseq = f.seq_mode ? M : 1, T = f.seq_mode ? 1 : M;
    SeqStateCache::Layer& sl = f.states.layers[layer];
    KF_TRY(kf_bias_act(f.ctx, s.mid, ak ? 1 : 0, m.rank_a, u + off[4], ldu, nullptr, 0, nullptr, 0, M, m.rank_a));
    KF_TRY(Lin(f, s.lat, nq, a2, s.mid, m.rank_a, M));
    KF_TRY(kf_gated_scan(f.ctx, s.y, nv, u + off[0], ldu, u + off[1], ldu, u + off[2], ldu, s.lat, nq, a2_b->data, nullptr, nullptr, 0, sl.state, sl.state_stride,
                         f.d_pos, f.d_slot, nseq, T, m.heads, m.heads, m.dim, m.vdim, 0, 0, m.tau, 0, 0.f, 1.0f / std::sqrt((float)m.dim)));
    KF_TRY(kf_group_rmsnorm_ex(f.ctx, s.act, ak, nv, nullptr, 0.f, s.y, nv, u + off[3], ldu, nullptr, 4, norm->data, 1, nullptr, M, nv, m.heads,
                               f.config.norm_rms_eps));
    KF_TRY(Lin(f, s.sub, f.config.n_embd, o, s.act, nv, M));
    return AddTo(f, s.sub, nullptr, M);
}

int PairMixer::cuInfer(int M, float* u, int ldu, const int* off) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MIXER_CARD& m = card;
    const MODEL_CARD& c = f.config;
    const int ak = c.compute_f32 ? 1 : 0, E = c.n_embd;
    const int nk = m.kv_heads * m.dim, nv = m.kv_heads * m.vdim, no = m.heads * m.vdim, Wd = m.lru_width;
    const int nseq = f.seq_mode ? M : 1, T = f.seq_mode ? 1 : M;
    SeqStateCache::Layer& sl = f.states.layers[layer];
    float* x = (float*)f.x;
    // left: this step's keys and values join the slot's rows, then attention over the rows 0 .. pos, gated, projected, normed into x
    KF_TRY(kf_kv_append(f.ctx, sl.rows, ak, sl.row_stride, u + off[1], ldu, nk, u + off[2], ldu, nv, f.d_pos, f.d_slot, M));
    // panels of one sequence with head sizes the tensor-core kernel takes go there; everything else (decode, odd sizes, 32-bit) to the general kernel
    if (!ak && f.panel_consecutive && f.seq_mode == 0 && M >= 16 && m.dim == m.vdim && (m.dim == 64 || m.dim == 128) && ldu % 2 == 0 && off[3] % 2 == 0)
        KF_TRY(kf_attn_bias_panel(f.ctx, s.act, s.y, u + off[0], ldu, u + off[3], ldu, sl.rows, sl.row_stride, r1->data, r2->data, f.d_pos, f.d_slot, M, m.heads,
                                  m.kv_heads, m.dim, c.max_seq_len, m.scale, m.qt_coef, m.qt_every));
    else
        KF_TRY(kf_attn_bias(f.ctx, s.act, ak, no, u + off[0], ldu, u + off[3], ldu, sl.rows, ak, sl.row_stride, r1->data, r2->data, f.d_pos, f.d_slot, M, m.heads,
                            m.kv_heads, m.dim, m.vdim, m.scale, m.qt_coef, m.qt_every, f.attn_hint));
    KF_TRY(Lin(f, s.sub, E, lo, s.act, no, M));
    KF_TRY(kf_group_rmsnorm(f.ctx, nullptr, 2, E, x, 0.5f, s.sub, E, nullptr, 0, nullptr, 0, lout->data, nullptr, M, E, 1, c.norm_rms_eps));
    // right: the convolved branch (its bias joins before the convolution, so the stored tail holds biased inputs), gates, recurrence
    KF_TRY(kf_bias_act(f.ctx, u + off[5], 1, ldu, u + off[5], ldu, rx_b->data, 0, nullptr, 0, M, Wd));
    KF_TRY(kf_conv1d(f.ctx, s.v, u, ldu, off[5], conv->data, conv_b->data, sl.tail, sl.tail_stride, f.d_pos, f.d_slot, nseq, T, Wd, m.lru_conv, 0));
    KF_TRY(kf_rglru(f.ctx, s.act, ak, Wd, s.lru_work, s.v, Wd, ra->data, ra_b->data, ri->data, ri_b->data, lam->data, 8.f, u + off[4], ldu, ry_b->data, sl.state,
                    sl.state_stride, f.d_pos, f.d_slot, nseq, T, Wd, m.lru_blocks));
    KF_TRY(Lin(f, s.sub, E, ro, s.act, Wd, M));
    KF_TRY(kf_group_rmsnorm(f.ctx, nullptr, 2, E, x, 0.5f, s.sub, E, nullptr, 0, nullptr, 0, rout->data, nullptr, M, E, 1, c.norm_rms_eps));
    return KF_OK;
}

int KvxFF::cuInfer(int M, const float* u, int ldu, int off) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const int E = f.config.n_embd, ak = f.config.compute_f32 ? 1 : 0;
    if (card.dense) {
        KF_TRY(kf_bias_act(f.ctx, s.h1, ak ? 1 : 0, card.ff, u + off, ldu, up_b->data, 1, nullptr, 0, M, card.ff));
        KF_TRY(Lin(f, s.sub, E, down, s.h1, card.ff, M));
        return AddTo(f, s.sub, down_b, M);
    }
    const int X = card.experts, top = card.top;
    KF_TRY(kf_moe_route_ex(f.ctx, s.idx, s.wgt, s.offsets, s.entry_slot, s.slot_row, s.slot_group, s.work, u + off, ldu, nullptr, M, X, top, 1));
    const void* const* tb = (const void* const*)tables;
    KF_TRY(kf_linear_grouped_act(f.ctx, s.h1, card.ff, tb, X, card.ff, E, s.hact, ak, E, s.offsets, s.slot_group, s.slot_row, M * top, 2));
    KF_TRY(kf_linear_grouped(f.ctx, s.yslots, E, tb + X, nullptr, X, E, card.ff, s.h1, ak, card.ff, s.offsets, s.slot_group, nullptr, M * top));
    KF_TRY(kf_moe_combine_ex(f.ctx, (float*)f.x, s.yslots, s.entry_slot, s.wgt, nullptr, nullptr, 0, M, E, top, 1));  // straight into the residual
    return KF_OK;
}

int KvxBlock::cuInfer(int M) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MODEL_CARD& c = f.config;
    const int E = c.n_embd, ak = c.compute_f32 ? 1 : 0, L = c.n_layers;
    float* x = (float*)f.x;
    // h = norm(x); one matmul for everything that reads h; the mixer and the feed-forward add their results to x (nothing reads x until
    // both are done: they work from h and the stacked projections)
    KF_TRY(kf_group_rmsnorm(f.ctx, s.hact, ak, E, nullptr, 0.f, x, E, nullptr, 0, nullptr, 0, norm1.w->data, nullptr, M, E, 1, norm1.eps));
    kf_tensor_desc d1 = {};
    d1.data_dev = cat.w, d1.rows = cat.rows, d1.cols = cat.cols, d1.type = KF_T_BF16, d1.group = 128;
    KF_TRY(kf_linear_g(f.ctx, s.u, cat.rows, &d1, s.hact, ak, E, M));
    size_t nmix = 0;
    if (delta) {
        KF_TRY(delta->cuInfer(M, s.u, cat.rows, off.data()));
        nmix = 6;
    } else if (gla) {
        KF_TRY(gla->cuInfer(M, s.u, cat.rows, off.data()));
        nmix = 5;
    } else {
        KF_TRY(pair->cuInfer(M, s.u, cat.rows, off.data()));
        nmix = 6;
    }
    if (ff) KF_TRY(ff->cuInfer(M, s.u, cat.rows, off[nmix]));
    if (c.side_dim > 0) {  // per-layer token input: gelu(gate x) * (this layer's slice of the token's side embedding) -> proj -> RMS norm -> x
        const int sd = c.side_dim;
        kf_tensor_desc dg = side_gate->Desc();
        KF_TRY(kf_linear_g(f.ctx, s.v, sd, &dg, x, 1, E, M));  // reads the fp32 residual as it is (no rounded copy) in both number formats
        KF_TRY(kf_token_gate(f.ctx, s.mid, ak, sd, s.v, sd, f.tensors["side.embed"]->data, L * sd, layer * sd, f.d_tokens, M, sd));
        KF_TRY(Lin(f, s.sub, E, side_proj, s.mid, sd, M));
        KF_TRY(kf_group_rmsnorm(f.ctx, nullptr, 2, E, x, 1.f, s.sub, E, nullptr, 0, nullptr, 0, side_norm->data, nullptr, M, E, 1, c.norm_rms_eps));
    }
    // depth average: this layer's result joins the history; the next layer reads the weighted sum of the history
    KF_TRY(kf_depth_mix(f.ctx, x, s.hist, (size_t)f.max_tokens * E, dwa->data, layer + 1, (size_t)M * E));
    return KF_OK;
}

static int ForwardKivorax(Fish& f, int M, bool want_logits) {
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MODEL_CARD& c = f.config;
    kf_tensor_desc de = f.embed.w->Desc();
    KF_TRY(kf_embed_f32_scaled(f.ctx, (float*)f.x, s.hist, &de, f.d_tokens, M, c.embed_scale));
    for (auto& n : f.blocks) KF_TRY(static_cast<KvxBlock*>(n.get())->cuInfer(M));
    if (want_logits && f.n_rows > 0) {
        const int R = f.n_rows, ak = c.compute_f32 ? 1 : 0;
        KF_TRY(kf_group_rmsnorm(f.ctx, s.head_in, ak, c.n_embd, nullptr, 0.f, (float*)f.x, c.n_embd, nullptr, 0, nullptr, 0, f.cls.norm.w->data, f.d_sel, R,
                                c.n_embd, 1, c.norm_rms_eps));
        KF_TRY(Lin(f, f.logits_f32, c.vocab, f.cls.proj.w, s.head_in, c.n_embd, R));
        KF_TRY(kf_f32_to_bf16(f.ctx, f.logits, f.logits_f32, (size_t)R * c.vocab));
    }
    return KF_OK;
}

const ARCH_ENTRY* KivoraxArch() {
    static const ARCH_ENTRY e = {"KIVORAX", ParseKivorax, BuildKivorax, ForwardKivorax, PrepareKivorax};
    return &e;
}

}  // namespace koifish
