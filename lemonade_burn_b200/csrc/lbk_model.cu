// The BitNet b1.58 decoder as a native runtime behind the C ABI: checkpoint loader, KV cache and the
// decode step, for hosts that want lb-model's `BitNet::{load, new_cache, forward}`
// (crates/lb-model/src/model.rs:149-232, 234-236, 305-374) without a tensor framework in between.
//
// Checkpoint: `config.json` + `model.lbt.safetensors` exactly as lb-convert writes them
// (crates/lb-convert/src/lib.rs:14-26: metadata format "lemonade-burn-ternary"; per linear
// `<name>.qweight` U8 [rows, padded(cols)/4] and `<name>.wscale` F32 [1]; norm gains F32; the tied
// embedding / LM head BF16). The packed weights go to the GPU as they are.
//
// Differences from the reference, all deliberate: the KV cache is bf16 with a fixed capacity
// (the reference grows an f32 cache, model.rs:245); several independent sequences can advance
// together (lbk_model_decode), which the reference cannot do. A call with several tokens of one
// sequence (a prompt) sends up to 4096 rows at a time through the projections (the tcgen05 GEMM
// above 16 rows) with causal attention over the cache, as the reference's forward does with
// m > 1. One decode step is recorded into a CUDA graph the first time a cache is used and
// replayed afterwards (the position lives in device memory).
#include <fcntl.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "lbk_internal.cuh"

namespace lbk {

namespace {

// ---- a small JSON reader (objects, arrays, strings, numbers, true/false/null) -----------------
struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;
    const Json *get(const char *key) const {
        for (const auto &kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
};

struct JsonParser {
    const char *p, *end;
    bool ok = true;
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool lit(const char *s) {
        const size_t n = strlen(s);
        if (static_cast<size_t>(end - p) >= n && memcmp(p, s, n) == 0) {
            p += n;
            return true;
        }
        return false;
    }
    std::string string() {
        std::string out;
        if (p >= end || *p != '"') {
            ok = false;
            return out;
        }
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u':  // keep the escape as text: tensor names and the fields read here are ASCII
                        out += "\\u";
                        break;
                    default: out += *p;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) ok = false;
        else ++p;
        return out;
    }
    Json value(int depth = 0) {
        Json j;
        ws();
        if (p >= end || depth > 64) {
            ok = false;
            return j;
        }
        if (*p == '{') {
            j.kind = Json::Obj;
            ++p;
            ws();
            if (p < end && *p == '}') {
                ++p;
                return j;
            }
            while (ok) {
                ws();
                std::string key = string();
                ws();
                if (!ok || p >= end || *p != ':') {
                    ok = false;
                    break;
                }
                ++p;
                j.obj.emplace_back(std::move(key), value(depth + 1));
                ws();
                if (p < end && *p == ',') {
                    ++p;
                    continue;
                }
                if (p < end && *p == '}') {
                    ++p;
                    break;
                }
                ok = false;
            }
        } else if (*p == '[') {
            j.kind = Json::Arr;
            ++p;
            ws();
            if (p < end && *p == ']') {
                ++p;
                return j;
            }
            while (ok) {
                j.arr.push_back(value(depth + 1));
                ws();
                if (p < end && *p == ',') {
                    ++p;
                    continue;
                }
                if (p < end && *p == ']') {
                    ++p;
                    break;
                }
                ok = false;
            }
        } else if (*p == '"') {
            j.kind = Json::Str;
            j.str = string();
        } else if (lit("true")) {
            j.kind = Json::Bool;
            j.b = true;
        } else if (lit("false")) {
            j.kind = Json::Bool;
        } else if (lit("null")) {
            j.kind = Json::Null;
        } else {
            char *e = nullptr;
            j.kind = Json::Num;
            j.num = strtod(p, &e);
            if (e == p || e > end) ok = false;
            else p = e;
        }
        return j;
    }
};

bool parse_json(const std::string &text, Json &out) {
    JsonParser ps{text.data(), text.data() + text.size()};
    out = ps.value();
    ps.ws();
    return ps.ok && ps.p == ps.end;
}

bool read_file(const std::string &path, std::string &out) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    std::string data;
    char buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) data.append(buf, n);
    fclose(f);
    out.swap(data);
    return true;
}

struct TensorEntry {
    std::string dtype;
    std::vector<size_t> shape;
    size_t begin = 0, end = 0;  // byte range inside the data section
};

}  // namespace

struct Model {
    Ctx *ctx = nullptr;
    lbk_model_config cfg{};
    size_t head_dim = 0;
    struct Layer {
        lbk_weight *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
        float *input_norm = nullptr, *post_attn_norm = nullptr, *attn_sub_norm = nullptr, *ffn_sub_norm = nullptr;
    };
    std::vector<Layer> layers;
    float *final_norm = nullptr;
    size_t prefill_rows = 0;    // prompt rows per pass (lbk_model_set_prefill_rows)
    uint16_t *embed = nullptr;  // bf16 [vocab][hidden], also the LM head (tied)
    float *cos = nullptr, *sin = nullptr;
    std::vector<void *> device_allocs;
    std::vector<lbk_weight *> weights;
    int rank = 0, world = 1;  // tensor-parallel shard this model holds (lbk_model_load_shard)
    lbk_load_stats stats{};
};

struct Cache {
    Model *model = nullptr;
    size_t b = 0, cap = 0, splits = 1;
    uint16_t *k = nullptr, *v = nullptr;  // [layers][b][kv_heads][cap][head_dim]
    int32_t *pos = nullptr;               // [b] cache length of every sequence, on the device
    int32_t *active = nullptr;            // [b] 1: the sequence takes part in the step (its position advances)
    std::vector<size_t> lens;             // the lengths again, on the host
    // work buffers of one step
    int32_t *tokens = nullptr, *next = nullptr, *counters = nullptr;
    float *x = nullptr, *x2 = nullptr, *n = nullptr, *q = nullptr, *kk = nullptr, *vv = nullptr, *attn = nullptr, *o = nullptr, *g = nullptr,
          *u = nullptr, *d = nullptr, *act = nullptr, *logits = nullptr, *scratch = nullptr;
    int8_t *q8 = nullptr;  // quantised input rows of the next projection (batches of 9 and more)
    float *qscale = nullptr;
    int32_t *qsum = nullptr;
    cudaGraphExec_t step = nullptr;
    std::vector<void *> device_allocs;
    // work buffers of the prompt path (lbk_model_forward with several tokens), sized for pf_rows rows
    size_t pf_rows = 0;
    std::vector<void *> pf_allocs;
    int32_t *pf_tokens = nullptr;
    float *pf_x = nullptr, *pf_n = nullptr, *pf_q = nullptr, *pf_k = nullptr, *pf_v = nullptr, *pf_attn = nullptr, *pf_o = nullptr, *pf_g = nullptr,
          *pf_u = nullptr, *pf_act = nullptr, *pf_d = nullptr, *pf_logits = nullptr;
    int8_t *pf_q8 = nullptr;   // quantised input rows of the next projection (lbk_norm_quant)
    float *pf_qscale = nullptr;
    int32_t *pf_qsum = nullptr;
};

// Continuous batching over one cache of `slots` sequences: what the reference's server would need in
// front of a batched decode step (its worker serves one request at a time,
// crates/lb-server/src/main.rs:92-166). Requests wait in a queue; a free slot takes the next one
// (its prompt goes through the prompt pass into that slot); every step advances all occupied slots
// by one greedy token (sample.rs:17-25) with the recorded decode step; a finished request frees
// its slot at once.
struct Request {
    uint64_t id = 0;
    std::vector<uint32_t> prompt, out;
    size_t max_new = 0;
    int32_t eos = -1;
    bool done = false;
    int slot = -1;
};

struct Batcher {
    Model *model = nullptr;
    Cache *cache = nullptr;
    std::deque<uint64_t> queue;
    std::map<uint64_t, Request> reqs;
    std::vector<uint64_t> slot_req;  // 0: the slot is free
    uint64_t next_id = 1;
};

namespace {

int dev_alloc(std::vector<void *> &owner, size_t bytes, void **out) {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail(LBK_ERR_NOMEM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    owner.push_back(p);
    *out = p;
    return LBK_OK;
}

// model.rs:213-230: inv_freq in f32, angle = pos as f32 * inv_freq (f32), sin/cos evaluated in f64,
// stored as f32, the 64 values repeated for both halves of the head.
void rope_tables(const lbk_model_config &c, size_t hd, std::vector<float> &cs, std::vector<float> &sn) {
    const size_t half = hd / 2, np = c.max_position_embeddings;
    cs.resize(np * hd);
    sn.resize(np * hd);
    std::vector<float> inv(half);
    for (size_t i = 0; i < half; ++i) inv[i] = static_cast<float>(1.0 / std::pow(static_cast<double>(c.rope_theta), (2.0 * i) / hd));
    for (size_t p = 0; p < np; ++p)
        for (size_t i = 0; i < half; ++i) {
            const float ang = static_cast<float>(p) * inv[i];
            const float cv = static_cast<float>(std::cos(static_cast<double>(ang))), sv = static_cast<float>(std::sin(static_cast<double>(ang)));
            cs[p * hd + i] = cs[p * hd + half + i] = cv;
            sn[p * hd + i] = sn[p * hd + half + i] = sv;
        }
}

size_t json_size(const Json *j, bool &ok) {
    if (!j || j->kind != Json::Num || j->num < 0) {
        ok = false;
        return 0;
    }
    return static_cast<size_t>(j->num);
}

// One decode step for cache->b sequences: the C++ twin of the Python mirror's BitNet.forward.
int enqueue_step(Model *m, Cache *c, cudaStream_t st) {
    lbk_ctx *h = reinterpret_cast<lbk_ctx *>(m->ctx);
    const lbk_model_config &cfg = m->cfg;
    const size_t b = c->b, H = cfg.hidden_size, I = cfg.intermediate_size, nh = cfg.num_attention_heads, kvh = cfg.num_key_value_heads,
                 hd = m->head_dim, L = cfg.num_hidden_layers;
    const float eps = cfg.rms_norm_eps;
    const bool pre_h = lbk_ternary_linear_pre_supported(b, H), pre_a = lbk_ternary_linear_pre_supported(b, nh * hd),
               pre_i = lbk_ternary_linear_pre_supported(b, I);
    const bool fused_norms = H % 4 == 0 && H <= 8192 && I % 4 == 0 && I <= 8192;
    const bool attn_fused = lbk_attn_decode_fused_supported(nh, kvh, hd, c->splits) != 0;
    const size_t layer_kv = b * kvh * c->cap * hd;
    float *x = c->x, *x2 = c->x2;
    auto add_norm = [&](float *xin, const float *y, const float *w) -> int {  // xin += y; n = rms_norm(xin) * w
        if (fused_norms) return lbk_add_rms_norm(h, xin, y, w, b, H, eps, c->n, st);
        LBK_TRY(lbk_add_inplace(h, xin, y, b * H, st));
        return lbk_rms_norm(h, xin, w, b, H, eps, c->n, st);
    };
    // From 9 sequences on every projection takes the quantise + GEMM path; the norm in front of it then
    // writes the quantised rows itself (lbk_norm_quant): no f32 copy, no quantise kernel. Same bits.
    const bool nq = b >= 9 && lbk_norm_quant_supported(H) && lbk_norm_quant_supported(I) && lbk_norm_quant_supported(nh * hd);
    auto norm_q = [&](int pre, float *xx, const float *yy, const float *w, size_t width) -> int {
        return lbk_norm_quant(h, pre, xx, yy, w, b, width, eps, c->q8, c->qscale, c->qsum, st);
    };
    auto proj_q = [&](const lbk_weight *const *ws, size_t nw, float *const *outs) -> int {
        return lbk_ternary_gemm_dev(h, ws, nw, c->q8, c->qscale, c->qsum, b, outs, nullptr, st);
    };
    LBK_TRY(lbk_embed_bf16(h, m->embed, c->tokens, b, H, x, st));
    bool have_d = false;  // c->d holds the previous layer's down projection, not yet added to x
    for (size_t li = 0; li < L; ++li) {
        const Model::Layer &l = m->layers[li];
        const lbk_weight *qkv[3] = {l.q, l.k, l.v};
        float *qkv_out[3] = {c->q, c->kk, c->vv};
        if (nq) {
            LBK_TRY(norm_q(have_d ? LBK_PRE_ADD_RMS : LBK_PRE_RMS, x, have_d ? c->d : nullptr, l.input_norm, H));
            LBK_TRY(proj_q(qkv, 3, qkv_out));
        } else if (!have_d) {
            if (pre_h) {
                LBK_TRY(lbk_ternary_linear_pre(h, LBK_PRE_RMS, x, nullptr, l.input_norm, eps, nullptr, b, qkv, 3, qkv_out, nullptr, st));
            } else {
                LBK_TRY(lbk_rms_norm(h, x, l.input_norm, b, H, eps, c->n, st));
                LBK_TRY(lbk_ternary_linear_n(h, c->n, b, qkv, 3, qkv_out, nullptr, st));
            }
        } else if (pre_h) {
            LBK_TRY(lbk_ternary_linear_pre(h, LBK_PRE_ADD_RMS, x, c->d, l.input_norm, eps, x2, b, qkv, 3, qkv_out, nullptr, st));
            std::swap(x, x2);
        } else {
            LBK_TRY(add_norm(x, c->d, l.input_norm));
            LBK_TRY(lbk_ternary_linear_n(h, c->n, b, qkv, 3, qkv_out, nullptr, st));
        }
        uint16_t *kc = c->k + li * layer_kv, *vc = c->v + li * layer_kv;
        if (attn_fused) {
            LBK_TRY(lbk_attn_decode_fused_seq(h, c->q, c->kk, c->vv, m->cos, m->sin, c->pos, b, nh, kvh, hd, c->cap, c->splits, kc, vc, c->scratch,
                                          c->counters, c->attn, st));
        } else {
            LBK_TRY(lbk_rope_kv_append_seq(h, c->q, c->kk, c->vv, m->cos, m->sin, c->pos, b, nh, kvh, hd, c->cap, kc, vc, st));
            LBK_TRY(lbk_attn_decode_seq(h, c->q, kc, vc, c->pos, b, nh, kvh, hd, c->cap, c->splits, c->scratch, c->attn, st));
        }
        const lbk_weight *ow[1] = {l.o};
        float *oo[1] = {c->o};
        if (nq) {
            const lbk_weight *gu[2] = {l.gate, l.up}, *dw[1] = {l.down};
            float *guo[2] = {c->g, c->u}, *dout[1] = {c->d};
            LBK_TRY(norm_q(LBK_PRE_RMS, c->attn, nullptr, l.attn_sub_norm, nh * hd));
            LBK_TRY(proj_q(ow, 1, oo));
            LBK_TRY(norm_q(LBK_PRE_ADD_RMS, x, c->o, l.post_attn_norm, H));
            LBK_TRY(proj_q(gu, 2, guo));
            LBK_TRY(norm_q(LBK_PRE_RELU2_MUL_RMS, c->g, c->u, l.ffn_sub_norm, I));
            LBK_TRY(proj_q(dw, 1, dout));
            have_d = true;
            continue;
        }
        if (pre_a) {
            LBK_TRY(lbk_ternary_linear_pre(h, LBK_PRE_RMS, c->attn, nullptr, l.attn_sub_norm, eps, nullptr, b, ow, 1, oo, nullptr, st));
        } else {
            LBK_TRY(lbk_rms_norm(h, c->attn, l.attn_sub_norm, b, nh * hd, eps, c->attn, st));
            LBK_TRY(lbk_ternary_linear_n(h, c->attn, b, ow, 1, oo, nullptr, st));
        }
        const lbk_weight *gu[2] = {l.gate, l.up};
        float *guo[2] = {c->g, c->u};
        if (pre_h) {
            LBK_TRY(lbk_ternary_linear_pre(h, LBK_PRE_ADD_RMS, x, c->o, l.post_attn_norm, eps, x2, b, gu, 2, guo, nullptr, st));
            std::swap(x, x2);
        } else {
            LBK_TRY(add_norm(x, c->o, l.post_attn_norm));
            LBK_TRY(lbk_ternary_linear_n(h, c->n, b, gu, 2, guo, nullptr, st));
        }
        const lbk_weight *dw[1] = {l.down};
        float *dout[1] = {c->d};
        if (pre_i) {
            LBK_TRY(lbk_ternary_linear_pre(h, LBK_PRE_RELU2_MUL_RMS, c->g, c->u, l.ffn_sub_norm, eps, nullptr, b, dw, 1, dout, nullptr, st));
        } else {
            if (fused_norms) {
                LBK_TRY(lbk_relu2_mul_rms_norm(h, c->g, c->u, l.ffn_sub_norm, b, I, eps, c->act, st));
            } else {
                LBK_TRY(lbk_relu2_mul(h, c->g, c->u, b * I, c->act, st));
                LBK_TRY(lbk_rms_norm(h, c->act, l.ffn_sub_norm, b, I, eps, c->act, st));
            }
            LBK_TRY(lbk_ternary_linear_n(h, c->act, b, dw, 1, dout, nullptr, st));
        }
        have_d = true;
    }
    if (have_d) LBK_TRY(add_norm(x, c->d, m->final_norm));
    else LBK_TRY(lbk_rms_norm(h, x, m->final_norm, b, H, eps, c->n, st));
    LBK_TRY(lbk_bf16_linear(h, c->n, b, m->embed, cfg.vocab_size, H, c->logits, st));
    LBK_TRY(lbk_argmax(h, c->logits, b, cfg.vocab_size, c->next, st));  // sample.rs:17-25
    LBK_TRY(lbk_advance_pos_seq(h, c->pos, c->active, b, st));
    return LBK_OK;
}

// Prompt rows per pass. More rows fill the GEMM's tile rounds better (a 4032-token prompt at 2B4T
// shapes: 41.3 ms at 1024 rows a pass, 34.8 at 2048, 30.6 at 4096); the work buffers grow with them
// (about 150 KB per row at those shapes, allocated for the rows a prompt really has).
// lbk_model_set_prefill_rows changes it per model.
constexpr size_t kPrefillChunk = 4096;
constexpr size_t kLogitRows = 128;      // rows of logits staged on the device at a time when every token's are wanted

int ensure_prefill_buffers(Model *m, Cache *c, size_t rows) {
    if (rows <= c->pf_rows) return LBK_OK;
    LBK_CUDA(cudaDeviceSynchronize());
    for (void *p : c->pf_allocs) cudaFree(p);
    c->pf_allocs.clear();
    c->pf_rows = 0;
    const lbk_model_config &cfg = m->cfg;
    const size_t H = cfg.hidden_size, I = cfg.intermediate_size, nh = cfg.num_attention_heads, kvh = cfg.num_key_value_heads, hd = m->head_dim;
    struct { void **p; size_t bytes; } bufs[] = {
        {reinterpret_cast<void **>(&c->pf_tokens), rows * 4}, {reinterpret_cast<void **>(&c->pf_x), rows * H * 4},
        {reinterpret_cast<void **>(&c->pf_n), rows * H * 4}, {reinterpret_cast<void **>(&c->pf_q), rows * nh * hd * 4},
        {reinterpret_cast<void **>(&c->pf_k), rows * kvh * hd * 4}, {reinterpret_cast<void **>(&c->pf_v), rows * kvh * hd * 4},
        {reinterpret_cast<void **>(&c->pf_attn), rows * nh * hd * 4}, {reinterpret_cast<void **>(&c->pf_o), rows * H * 4},
        {reinterpret_cast<void **>(&c->pf_g), rows * I * 4}, {reinterpret_cast<void **>(&c->pf_u), rows * I * 4},
        {reinterpret_cast<void **>(&c->pf_act), rows * I * 4}, {reinterpret_cast<void **>(&c->pf_d), rows * H * 4},
        {reinterpret_cast<void **>(&c->pf_logits), kLogitRows * cfg.vocab_size * 4},
        {reinterpret_cast<void **>(&c->pf_q8), rows * (std::max(std::max(H, I), nh * hd) + 127) / 128 * 128},
        {reinterpret_cast<void **>(&c->pf_qscale), rows * 4}, {reinterpret_cast<void **>(&c->pf_qsum), rows * 4}};
    for (auto &bf : bufs) LBK_TRY(dev_alloc(c->pf_allocs, bf.bytes, bf.p));
    c->pf_rows = rows;
    return LBK_OK;
}

// `n` (at most the model's prefill_rows) consecutive tokens of sequence `seq` of the cache in one pass: the
// projections see n token rows (the tcgen05 GEMM above 16 rows), attention is causal over the cache
// (model.rs:305-374 with m = n). Logits of every row (`all_logits`) or of the last one go to host
// memory; `next_out` (host) receives the greedy token after the last row (sample.rs:17-25).
// Synchronous.
int prefill_chunk(Model *m, Cache *c, size_t seq, const uint32_t *tokens, size_t n, int all_logits, float *logits_out, int32_t *next_out = nullptr) {
    Ctx *ctx = m->ctx;
    lbk_ctx *h = reinterpret_cast<lbk_ctx *>(ctx);
    cudaStream_t st = ctx->own_stream;
    const lbk_model_config &cfg = m->cfg;
    const size_t H = cfg.hidden_size, I = cfg.intermediate_size, nh = cfg.num_attention_heads, kvh = cfg.num_key_value_heads, hd = m->head_dim,
                 L = cfg.num_hidden_layers, V = cfg.vocab_size;
    const float eps = cfg.rms_norm_eps;
    LBK_TRY(ensure_prefill_buffers(m, c, n));
    std::vector<int32_t> toks(n);
    for (size_t i = 0; i < n; ++i) toks[i] = static_cast<int32_t>(tokens[i]);
    LBK_CUDA(cudaMemcpyAsync(c->pf_tokens, toks.data(), n * 4, cudaMemcpyHostToDevice, st));
    LBK_CUDA(cudaStreamSynchronize(st));  // `toks` is pageable host memory that goes away
    const bool fused_h = H % 4 == 0 && H <= 8192, fused_i = I % 4 == 0 && I <= 8192;
    auto add_norm = [&](float *x, const float *y, const float *w) -> int {  // x += y; pf_n = rms_norm(x) * w
        if (fused_h) return lbk_add_rms_norm(h, x, y, w, n, H, eps, c->pf_n, st);
        LBK_TRY(lbk_add_inplace(h, x, y, n * H, st));
        return lbk_rms_norm(h, x, w, n, H, eps, c->pf_n, st);
    };
    const size_t layer_kv = c->b * kvh * c->cap * hd;
    // From 9 rows on every projection takes the GEMM path, whose input is the quantised rows: the norm
    // in front of a projection then writes those directly (lbk_norm_quant) and the f32 copy of the
    // normalised rows, with the quantise kernel that would read it back, goes away. Same bits.
    const bool nq = n >= 9 && lbk_norm_quant_supported(H) && lbk_norm_quant_supported(I) && lbk_norm_quant_supported(nh * hd);
    auto norm_q = [&](int pre, float *x, const float *y, const float *w, size_t width) -> int {
        return lbk_norm_quant(h, pre, x, y, w, n, width, eps, c->pf_q8, c->pf_qscale, c->pf_qsum, st);
    };
    auto project = [&](const float *x_f32, const lbk_weight *const *ws, size_t nw, float *const *outs) -> int {
        if (nq) return lbk_ternary_gemm_dev(h, ws, nw, c->pf_q8, c->pf_qscale, c->pf_qsum, n, outs, nullptr, st);
        return lbk_ternary_linear_n(h, x_f32, n, ws, nw, outs, nullptr, st);
    };
    LBK_TRY(lbk_embed_bf16(h, m->embed, c->pf_tokens, n, H, c->pf_x, st));
    if (nq) LBK_TRY(norm_q(LBK_PRE_RMS, c->pf_x, nullptr, m->layers[0].input_norm, H));
    else LBK_TRY(lbk_rms_norm(h, c->pf_x, m->layers[0].input_norm, n, H, eps, c->pf_n, st));
    for (size_t li = 0; li < L; ++li) {
        const Model::Layer &l = m->layers[li];
        const lbk_weight *qkv[3] = {l.q, l.k, l.v};
        float *qkv_out[3] = {c->pf_q, c->pf_k, c->pf_v};
        LBK_TRY(project(c->pf_n, qkv, 3, qkv_out));
        uint16_t *kc = c->k + li * layer_kv, *vc = c->v + li * layer_kv;
        LBK_TRY(lbk_rope_kv_append_rows(h, c->pf_q, c->pf_k, c->pf_v, m->cos, m->sin, c->pos + seq, n, nh, kvh, hd, c->cap, seq, kc, vc, st));
        LBK_TRY(lbk_attn_prefill(h, c->pf_q, kc, vc, c->pos + seq, n, nh, kvh, hd, c->cap, seq, c->pf_attn, st));
        if (nq) LBK_TRY(norm_q(LBK_PRE_RMS, c->pf_attn, nullptr, l.attn_sub_norm, nh * hd));
        else LBK_TRY(lbk_rms_norm(h, c->pf_attn, l.attn_sub_norm, n, nh * hd, eps, c->pf_attn, st));
        const lbk_weight *ow[1] = {l.o};
        float *oo[1] = {c->pf_o};
        LBK_TRY(project(c->pf_attn, ow, 1, oo));
        if (nq) LBK_TRY(norm_q(LBK_PRE_ADD_RMS, c->pf_x, c->pf_o, l.post_attn_norm, H));
        else LBK_TRY(add_norm(c->pf_x, c->pf_o, l.post_attn_norm));
        const lbk_weight *gu[2] = {l.gate, l.up};
        float *guo[2] = {c->pf_g, c->pf_u};
        LBK_TRY(project(c->pf_n, gu, 2, guo));
        if (nq) {
            LBK_TRY(norm_q(LBK_PRE_RELU2_MUL_RMS, c->pf_g, c->pf_u, l.ffn_sub_norm, I));
        } else if (fused_i) {
            LBK_TRY(lbk_relu2_mul_rms_norm(h, c->pf_g, c->pf_u, l.ffn_sub_norm, n, I, eps, c->pf_act, st));
        } else {
            LBK_TRY(lbk_relu2_mul(h, c->pf_g, c->pf_u, n * I, c->pf_act, st));
            LBK_TRY(lbk_rms_norm(h, c->pf_act, l.ffn_sub_norm, n, I, eps, c->pf_act, st));
        }
        const lbk_weight *dw[1] = {l.down};
        float *dout[1] = {c->pf_d};
        LBK_TRY(project(c->pf_act, dw, 1, dout));
        if (nq && li + 1 < L) LBK_TRY(norm_q(LBK_PRE_ADD_RMS, c->pf_x, c->pf_d, m->layers[li + 1].input_norm, H));
        else LBK_TRY(add_norm(c->pf_x, c->pf_d, li + 1 < L ? m->layers[li + 1].input_norm : m->final_norm));
    }
    // pf_n holds the final norm of every row
    if (logits_out) {
        if (all_logits) {
            for (size_t r0 = 0; r0 < n; r0 += kLogitRows) {
                const size_t rows = n - r0 < kLogitRows ? n - r0 : kLogitRows;
                LBK_TRY(lbk_bf16_linear(h, c->pf_n + r0 * H, rows, m->embed, V, H, c->pf_logits, st));
                LBK_CUDA(cudaMemcpyAsync(logits_out + r0 * V, c->pf_logits, rows * V * 4, cudaMemcpyDeviceToHost, st));
                LBK_CUDA(cudaStreamSynchronize(st));  // the staging rows are reused by the next pass
            }
        } else {
            LBK_TRY(lbk_bf16_linear(h, c->pf_n + (n - 1) * H, 1, m->embed, V, H, c->pf_logits, st));
            LBK_CUDA(cudaMemcpyAsync(logits_out, c->pf_logits, V * 4, cudaMemcpyDeviceToHost, st));
        }
    }
    if (next_out) {
        if (!logits_out || all_logits) LBK_TRY(lbk_bf16_linear(h, c->pf_n + (n - 1) * H, 1, m->embed, V, H, c->pf_logits, st));
        LBK_TRY(lbk_argmax(h, c->pf_logits, 1, V, c->pf_tokens, st));  // the token buffer is free again
        LBK_CUDA(cudaMemcpyAsync(next_out, c->pf_tokens, 4, cudaMemcpyDeviceToHost, st));
    }
    const int32_t new_len = static_cast<int32_t>(c->lens[seq] + n);
    LBK_CUDA(cudaStreamSynchronize(st));
    LBK_CUDA(cudaMemcpy(c->pos + seq, &new_len, 4, cudaMemcpyHostToDevice));
    c->lens[seq] += n;
    return LBK_OK;
}

// Records the step into a graph on the context's own stream (a few eager steps first: the library's
// scratch buffers must exist before anything is captured; those steps run on a scratch position).
int ensure_graph(Model *m, Cache *c) {
    if (c->step) return LBK_OK;
    Ctx *ctx = m->ctx;
    cudaStream_t st = ctx->own_stream;
    std::vector<int32_t> saved(c->b);
    LBK_CUDA(cudaMemcpy(saved.data(), c->pos, c->b * 4, cudaMemcpyDeviceToHost));
    LBK_TRY(enqueue_step(m, c, st));  // eager warm-up: writes the K/V rows of the saved positions, which the real step rewrites
    LBK_CUDA(cudaStreamSynchronize(st));
    LBK_CUDA(cudaMemcpy(c->pos, saved.data(), c->b * 4, cudaMemcpyHostToDevice));
    const uint64_t before = ctx->launches;
    LBK_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    const int status = enqueue_step(m, c, st);
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(st, &graph);
    ctx->launches = before;  // recording is not launching
    if (status != LBK_OK) {
        if (graph) cudaGraphDestroy(graph);
        return status;
    }
    if (e != cudaSuccess) return fail(LBK_ERR_CUDA, "capture of the decode step failed: %s", cudaGetErrorString(e));
    const cudaError_t ei = cudaGraphInstantiate(&c->step, graph, 0);
    cudaGraphDestroy(graph);
    if (ei != cudaSuccess) return fail(LBK_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(ei));
    return LBK_OK;
}

}  // namespace

}  // namespace lbk

using namespace lbk;

extern "C" {

int lbk_model_free(lbk_model *mp) {
    if (!mp) return LBK_OK;
    Model *m = reinterpret_cast<Model *>(mp);
    cudaSetDevice(m->ctx->device);
    cudaDeviceSynchronize();
    for (lbk_weight *w : m->weights) lbk_weight_free(w);
    for (void *p : m->device_allocs) cudaFree(p);
    delete m;
    return LBK_OK;
}

// ---- loader ------------------------------------------------------------------------------------
// The reference maps the file and copies every tensor into a framework tensor, which doubles its
// resident memory while loading (crates/lb-model/src/model.rs:172-183, docs/BENCHMARKS.md:57-59).
// Here tensor bytes go file -> one of two pinned staging buffers (pread) -> device (one
// cudaMemcpyAsync / cudaMemcpy2DAsync per piece on the context's stream); a buffer is refilled while
// the other one's copy is in flight. The host never holds more than the two buffers, whatever the
// model's size. All packed weights live in ONE device arena (256-byte aligned slices, wrapped as
// weights without a copy).
//
// Tensor parallel (rank, world): q/k/v/gate/up keep their row range [rank*rows/world, ...), which is a
// contiguous byte range of the file (rows are contiguous in the lb-ternary layout, pack.rs:46-49);
// o/down keep a column range that is a multiple of 128 columns, i.e. bytes [rank*rb/world, ...) of
// every packed row, cut out by a strided copy from the staging buffer. Norm gains, the embedding
// (also the head; a rank uses vocabulary rows [rank*V/world, ...) of it) and the RoPE tables are
// whole on every rank.
namespace {

constexpr size_t kStageBytes = 32u << 20;

struct Stager {
    int fd = -1;
    size_t file_size = 0, data0 = 0;
    cudaStream_t st = nullptr;
    unsigned char *buf[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    bool busy[2] = {false, false};
    int next = 0;
    size_t bytes_read = 0, bytes_to_device = 0;
    ~Stager() {
        for (int i = 0; i < 2; ++i) {
            if (busy[i]) cudaEventSynchronize(done[i]);
            if (done[i]) cudaEventDestroy(done[i]);
            if (buf[i]) cudaFreeHost(buf[i]);
        }
        if (fd >= 0) close(fd);
    }
    int init(cudaStream_t stream) {
        st = stream;
        for (int i = 0; i < 2; ++i) {
            cudaError_t e = cudaMallocHost(reinterpret_cast<void **>(&buf[i]), kStageBytes);
            if (e != cudaSuccess) return fail(LBK_ERR_NOMEM, "pinned staging buffer: %s", cudaGetErrorString(e));
            LBK_CUDA(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
        }
        return LBK_OK;
    }
    int acquire(int *slot) {
        const int s = next;
        next ^= 1;
        if (busy[s]) {
            LBK_CUDA(cudaEventSynchronize(done[s]));
            busy[s] = false;
        }
        *slot = s;
        return LBK_OK;
    }
    int fill(int s, size_t file_off, size_t n, const char *what) {
        if (file_off + n > file_size) return fail(LBK_ERR_INVALID, "the file is truncated: %s needs bytes up to %zu, the file has %zu", what, file_off + n, file_size);
        size_t got = 0;
        while (got < n) {
            const ssize_t r = pread(fd, buf[s] + got, n - got, static_cast<off_t>(file_off + got));
            if (r <= 0) return fail(LBK_ERR_INVALID, "cannot read %s (%zu of %zu bytes)", what, got, n);
            got += static_cast<size_t>(r);
        }
        bytes_read += n;
        return LBK_OK;
    }
    int release(int s) {
        LBK_CUDA(cudaEventRecord(done[s], st));
        busy[s] = true;
        return LBK_OK;
    }
    // `n` contiguous bytes at data offset `off` -> dst
    int copy_linear(size_t off, size_t n, void *dst, const char *what) {
        for (size_t o = 0; o < n; o += kStageBytes) {
            const size_t len = n - o < kStageBytes ? n - o : kStageBytes;
            int s;
            LBK_TRY(acquire(&s));
            LBK_TRY(fill(s, data0 + off + o, len, what));
            LBK_CUDA(cudaMemcpyAsync(static_cast<char *>(dst) + o, buf[s], len, cudaMemcpyHostToDevice, st));
            bytes_to_device += len;
            LBK_TRY(release(s));
        }
        return LBK_OK;
    }
    // bytes [c0, c0 + width) of each of `rows` rows of pitch `pitch` starting at data offset `off` -> dst (pitch = width)
    int copy_columns(size_t off, size_t rows, size_t pitch, size_t c0, size_t width, void *dst, const char *what) {
        const size_t rows_per = kStageBytes / pitch;
        if (rows_per == 0) return fail(LBK_ERR_UNSUPPORTED, "%s: a row of %zu bytes does not fit the staging buffer", what, pitch);
        for (size_t r = 0; r < rows; r += rows_per) {
            const size_t nr = rows - r < rows_per ? rows - r : rows_per;
            int s;
            LBK_TRY(acquire(&s));
            LBK_TRY(fill(s, data0 + off + r * pitch, nr * pitch, what));
            LBK_CUDA(cudaMemcpy2DAsync(static_cast<char *>(dst) + r * width, width, buf[s] + c0, pitch, width, nr, cudaMemcpyHostToDevice, st));
            bytes_to_device += nr * width;
            LBK_TRY(release(s));
        }
        return LBK_OK;
    }
};

double now_seconds() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return static_cast<double>(ts.tv_sec) + 1e-9 * static_cast<double>(ts.tv_nsec);
}

int load_impl(lbk_ctx *c, const char *directory, int rank, int world, lbk_model **out) {
    if (!c || !directory || !out) return fail(LBK_ERR_INVALID, "lbk_model_load: null argument");
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world) return fail(LBK_ERR_INVALID, "rank %d of %d", rank, world);
    const double t0 = now_seconds();
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    LBK_CUDA(cudaSetDevice(ctx->device));
    const std::string dir(directory);
    std::string text;
    if (!read_file(dir + "/config.json", text)) return fail(LBK_ERR_INVALID, "cannot read %s/config.json", directory);
    Json cj;
    if (!parse_json(text, cj) || cj.kind != Json::Obj) return fail(LBK_ERR_INVALID, "%s/config.json is not a JSON object", directory);
    std::unique_ptr<Model, int (*)(Model *)> model(new Model(), [](Model *m) { return lbk_model_free(reinterpret_cast<lbk_model *>(m)); });
    Model *m = model.get();
    m->ctx = ctx;
    m->rank = rank;
    m->world = world;
    m->prefill_rows = kPrefillChunk;
    bool ok = true;
    lbk_model_config &cfg = m->cfg;
    cfg.hidden_size = json_size(cj.get("hidden_size"), ok);
    cfg.intermediate_size = json_size(cj.get("intermediate_size"), ok);
    cfg.num_attention_heads = json_size(cj.get("num_attention_heads"), ok);
    cfg.num_key_value_heads = json_size(cj.get("num_key_value_heads"), ok);
    cfg.num_hidden_layers = json_size(cj.get("num_hidden_layers"), ok);
    cfg.vocab_size = json_size(cj.get("vocab_size"), ok);
    cfg.max_position_embeddings = json_size(cj.get("max_position_embeddings"), ok);
    const Json *je = cj.get("rms_norm_eps"), *jt = cj.get("rope_theta");
    if (!je || je->kind != Json::Num || !jt || jt->kind != Json::Num) ok = false;
    if (!ok) return fail(LBK_ERR_INVALID, "%s/config.json: a required field is missing or not a number", directory);
    cfg.rms_norm_eps = static_cast<float>(je->num);
    cfg.rope_theta = static_cast<float>(jt->num);
    const Json *jb = cj.get("bos_token_id");
    cfg.bos_token_id = jb && jb->kind == Json::Num ? static_cast<int>(jb->num) : 0;
    // model.rs:151-153: only the relu2, tied-embedding family
    // (both fields are required members of the reference's Config, model.rs:22-36: a file without them does not load there either)
    const Json *ja = cj.get("hidden_act"), *jtie = cj.get("tie_word_embeddings");
    if (!ja || !jtie) return fail(LBK_ERR_INVALID, "%s/config.json: missing field %s", directory, !ja ? "hidden_act" : "tie_word_embeddings");
    if (!(ja->kind == Json::Str && ja->str == "relu2")) return fail(LBK_ERR_UNSUPPORTED, "unsupported config: hidden_act must be relu2");
    if (!(jtie->kind == Json::Bool && jtie->b)) return fail(LBK_ERR_UNSUPPORTED, "unsupported config: tie_word_embeddings must be true");
    if (!cfg.num_attention_heads || !cfg.num_key_value_heads || cfg.hidden_size % cfg.num_attention_heads ||
        cfg.num_attention_heads % cfg.num_key_value_heads || !cfg.num_hidden_layers || !cfg.max_position_embeddings)
        return fail(LBK_ERR_INVALID, "config.json: inconsistent head counts or sizes");
    m->head_dim = cfg.hidden_size / cfg.num_attention_heads;
    if (m->head_dim != 128) return fail(LBK_ERR_UNSUPPORTED, "the attention kernels are built for head_dim 128, this model has %zu", m->head_dim);
    const size_t H = cfg.hidden_size, I = cfg.intermediate_size, hd = m->head_dim, W = static_cast<size_t>(world);
    if (world > 1 && (cfg.num_key_value_heads % W || I % (128 * W) || (cfg.num_attention_heads * hd) % (128 * W) || cfg.vocab_size % W))
        return fail(LBK_ERR_UNSUPPORTED, "%d ranks do not divide this model: KV heads %zu, intermediate %zu and attention width %zu (in blocks of 128 columns), vocabulary %zu",
                    world, cfg.num_key_value_heads, I, cfg.num_attention_heads * hd, cfg.vocab_size);

    // ---- model.lbt.safetensors: u64 header length, JSON header, data -------------------------
    const std::string path = dir + "/model.lbt.safetensors";
    Stager sg;
    sg.fd = open(path.c_str(), O_RDONLY);
    if (sg.fd < 0) return fail(LBK_ERR_INVALID, "cannot open %s", path.c_str());
    struct stat sb;
    if (fstat(sg.fd, &sb) != 0) return fail(LBK_ERR_INVALID, "cannot stat %s", path.c_str());
    sg.file_size = static_cast<size_t>(sb.st_size);
    unsigned char lenb[8];
    if (sg.file_size < 8 || pread(sg.fd, lenb, 8, 0) != 8) return fail(LBK_ERR_INVALID, "%s: truncated", path.c_str());
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | lenb[i];
    if (hlen == 0 || hlen > (100u << 20)) return fail(LBK_ERR_INVALID, "%s: implausible header length %llu", path.c_str(), static_cast<unsigned long long>(hlen));
    if (8 + hlen > sg.file_size) return fail(LBK_ERR_INVALID, "%s: truncated header", path.c_str());
    std::string header(hlen, '\0');
    if (pread(sg.fd, &header[0], hlen, 8) != static_cast<ssize_t>(hlen)) return fail(LBK_ERR_INVALID, "%s: truncated header", path.c_str());
    Json hj;
    if (!parse_json(header, hj) || hj.kind != Json::Obj) return fail(LBK_ERR_INVALID, "%s: header is not a JSON object", path.c_str());
    const Json *meta = hj.get("__metadata__");
    const Json *fmt = meta ? meta->get("format") : nullptr;
    if (!fmt || fmt->kind != Json::Str || fmt->str != "lemonade-burn-ternary")  // model.rs:158-161
        return fail(LBK_ERR_INVALID, "%s is not a lemonade-burn ternary file (format=%s)", path.c_str(), fmt && fmt->kind == Json::Str ? fmt->str.c_str() : "none");
    std::map<std::string, TensorEntry> entries;
    for (const auto &kv : hj.obj) {
        if (kv.first == "__metadata__") continue;
        const Json &t = kv.second;
        const Json *dt = t.get("dtype"), *sh = t.get("shape"), *off = t.get("data_offsets");
        if (!dt || dt->kind != Json::Str || !sh || sh->kind != Json::Arr || !off || off->kind != Json::Arr || off->arr.size() != 2)
            return fail(LBK_ERR_INVALID, "%s: malformed entry %s", path.c_str(), kv.first.c_str());
        TensorEntry e;
        e.dtype = dt->str;
        for (const Json &d : sh->arr) e.shape.push_back(static_cast<size_t>(d.num));
        e.begin = static_cast<size_t>(off->arr[0].num);
        e.end = static_cast<size_t>(off->arr[1].num);
        if (e.end < e.begin) return fail(LBK_ERR_INVALID, "%s: malformed offsets of %s", path.c_str(), kv.first.c_str());
        entries[kv.first] = e;
    }
    sg.data0 = static_cast<size_t>(8 + hlen);
    LBK_TRY(sg.init(ctx->own_stream));
    auto find_tensor = [&](const std::string &name, const char *dtype, size_t elems, size_t elem_bytes, const TensorEntry **e_out) -> int {
        auto it = entries.find(name);
        if (it == entries.end()) return fail(LBK_ERR_INVALID, "%s: tensor %s is missing", path.c_str(), name.c_str());
        const TensorEntry &e = it->second;
        size_t n = 1;
        for (size_t d : e.shape) n *= d;
        if (e.dtype != dtype || n != elems || e.end - e.begin != elems * elem_bytes)
            return fail(LBK_ERR_SHAPE, "%s: %s has dtype %s and %zu elements, expected %s and %zu", path.c_str(), name.c_str(), e.dtype.c_str(), n, dtype, elems);
        if (sg.data0 + e.end > sg.file_size)
            return fail(LBK_ERR_INVALID, "%s is truncated: %s ends at byte %zu, the file has %zu", path.c_str(), name.c_str(), sg.data0 + e.end, sg.file_size);
        *e_out = &e;
        return LBK_OK;
    };
    // norm gains (model.rs:165: F32) share one small arena
    const size_t L = cfg.num_hidden_layers;
    float *norms = nullptr;
    LBK_TRY(dev_alloc(m->device_allocs, (L * (3 * H + I) + H) * 4, reinterpret_cast<void **>(&norms)));
    size_t norm_off = 0;
    auto load_vec = [&](const std::string &name, size_t elems, float **dst) -> int {
        const TensorEntry *e;
        LBK_TRY(find_tensor(name, "F32", elems, 4, &e));
        *dst = norms + norm_off;
        norm_off += elems;
        return sg.copy_linear(e->begin, elems * 4, *dst, name.c_str());
    };
    // one arena for every packed matrix of this rank
    struct Lin { const char *name; size_t rows, cols; bool split_cols; };
    const Lin lins[7] = {{".self_attn.q_proj", cfg.num_attention_heads * hd, H, false}, {".self_attn.k_proj", cfg.num_key_value_heads * hd, H, false},
                         {".self_attn.v_proj", cfg.num_key_value_heads * hd, H, false}, {".self_attn.o_proj", H, cfg.num_attention_heads * hd, true},
                         {".mlp.gate_proj", I, H, false}, {".mlp.up_proj", I, H, false}, {".mlp.down_proj", H, I, true}};
    size_t arena_bytes = 0;
    for (const Lin &ln : lins) {
        const size_t rows = ln.split_cols ? ln.rows : ln.rows / W, cols = ln.split_cols ? ln.cols / W : ln.cols;
        arena_bytes += (rows * lbk_row_bytes(cols) + 255) / 256 * 256;
    }
    arena_bytes *= L;
    unsigned char *arena = nullptr;
    LBK_TRY(dev_alloc(m->device_allocs, arena_bytes, reinterpret_cast<void **>(&arena)));
    size_t arena_off = 0;
    m->layers.resize(L);
    for (size_t i = 0; i < L; ++i) {
        const std::string p = "model.layers." + std::to_string(i);
        Model::Layer &l = m->layers[i];
        LBK_TRY(load_vec(p + ".input_layernorm.weight", H, &l.input_norm));
        LBK_TRY(load_vec(p + ".post_attention_layernorm.weight", H, &l.post_attn_norm));
        LBK_TRY(load_vec(p + ".self_attn.attn_sub_norm.weight", H, &l.attn_sub_norm));
        LBK_TRY(load_vec(p + ".mlp.ffn_sub_norm.weight", I, &l.ffn_sub_norm));
        lbk_weight **dst[7] = {&l.q, &l.k, &l.v, &l.o, &l.gate, &l.up, &l.down};
        for (int k = 0; k < 7; ++k) {
            const Lin &ln = lins[k];
            const std::string name = p + ln.name;
            const TensorEntry *es, *ew;
            LBK_TRY(find_tensor(name + ".wscale", "F32", 1, 4, &es));
            float scale = 0.0f;
            if (pread(sg.fd, &scale, 4, static_cast<off_t>(sg.data0 + es->begin)) != 4) return fail(LBK_ERR_INVALID, "cannot read %s.wscale", name.c_str());
            const size_t rb = lbk_row_bytes(ln.cols);
            LBK_TRY(find_tensor(name + ".qweight", "U8", ln.rows * rb, 1, &ew));
            unsigned char *dev = arena + arena_off;
            size_t rows = ln.rows, cols = ln.cols;
            if (!ln.split_cols) {
                rows = ln.rows / W;
                LBK_TRY(sg.copy_linear(ew->begin + static_cast<size_t>(rank) * rows * rb, rows * rb, dev, name.c_str()));
            } else if (world == 1) {
                LBK_TRY(sg.copy_linear(ew->begin, rows * rb, dev, name.c_str()));
            } else {
                cols = ln.cols / W;
                const size_t width = rb / W;
                LBK_TRY(sg.copy_columns(ew->begin, rows, rb, static_cast<size_t>(rank) * width, width, dev, name.c_str()));
            }
            arena_off += (rows * lbk_row_bytes(cols) + 255) / 256 * 256;
            LBK_TRY(lbk_weight_wrap(c, rows, cols, dev, scale, dst[k]));
            m->weights.push_back(*dst[k]);
        }
    }
    LBK_TRY(load_vec("model.norm.weight", H, &m->final_norm));
    const TensorEntry *ee;
    LBK_TRY(find_tensor("model.embed_tokens.weight", "BF16", cfg.vocab_size * H, 2, &ee));  // model.rs:204
    LBK_TRY(dev_alloc(m->device_allocs, cfg.vocab_size * H * 2, reinterpret_cast<void **>(&m->embed)));
    LBK_TRY(sg.copy_linear(ee->begin, cfg.vocab_size * H * 2, m->embed, "model.embed_tokens.weight"));
    std::vector<float> cs, sn;
    rope_tables(cfg, hd, cs, sn);
    LBK_TRY(dev_alloc(m->device_allocs, cs.size() * 4, reinterpret_cast<void **>(&m->cos)));
    LBK_TRY(dev_alloc(m->device_allocs, sn.size() * 4, reinterpret_cast<void **>(&m->sin)));
    LBK_CUDA(cudaMemcpyAsync(m->cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, ctx->own_stream));
    LBK_CUDA(cudaMemcpyAsync(m->sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice, ctx->own_stream));
    LBK_CUDA(cudaStreamSynchronize(ctx->own_stream));  // also: `cs`, `sn` and the staging buffers go away now
    m->stats.seconds = now_seconds() - t0;
    m->stats.bytes_read = sg.bytes_read;
    m->stats.bytes_to_device = sg.bytes_to_device;
    m->stats.staging_bytes = 2 * kStageBytes;
    *out = reinterpret_cast<lbk_model *>(model.release());
    return LBK_OK;
}

}  // namespace

int lbk_model_load(lbk_ctx *c, const char *directory, lbk_model **out) { return load_impl(c, directory, 0, 1, out); }

int lbk_model_load_shard(lbk_ctx *c, const char *directory, int rank, int world, lbk_model **out) { return load_impl(c, directory, rank, world, out); }

int lbk_model_load_stats(const lbk_model *mp, lbk_load_stats *out) {
    if (!mp || !out) return fail(LBK_ERR_INVALID, "lbk_model_load_stats: null argument");
    *out = reinterpret_cast<const Model *>(mp)->stats;
    return LBK_OK;
}

const lbk_weight *lbk_model_linear(const lbk_model *mp, size_t layer, int which) {
    const Model *m = reinterpret_cast<const Model *>(mp);
    if (!m || layer >= m->layers.size()) return nullptr;
    const Model::Layer &l = m->layers[layer];
    switch (which) {
        case LBK_LIN_Q: return l.q;
        case LBK_LIN_K: return l.k;
        case LBK_LIN_V: return l.v;
        case LBK_LIN_O: return l.o;
        case LBK_LIN_GATE: return l.gate;
        case LBK_LIN_UP: return l.up;
        case LBK_LIN_DOWN: return l.down;
        default: return nullptr;
    }
}

const float *lbk_model_norm(const lbk_model *mp, size_t layer, int which) {
    const Model *m = reinterpret_cast<const Model *>(mp);
    if (!m) return nullptr;
    if (which == LBK_NORM_FINAL) return m->final_norm;
    if (layer >= m->layers.size()) return nullptr;
    const Model::Layer &l = m->layers[layer];
    switch (which) {
        case LBK_NORM_INPUT: return l.input_norm;
        case LBK_NORM_POST_ATTN: return l.post_attn_norm;
        case LBK_NORM_ATTN_SUB: return l.attn_sub_norm;
        case LBK_NORM_FFN_SUB: return l.ffn_sub_norm;
        default: return nullptr;
    }
}

const uint16_t *lbk_model_embedding(const lbk_model *mp) { return mp ? reinterpret_cast<const Model *>(mp)->embed : nullptr; }
const float *lbk_model_rope_cos(const lbk_model *mp) { return mp ? reinterpret_cast<const Model *>(mp)->cos : nullptr; }
const float *lbk_model_rope_sin(const lbk_model *mp) { return mp ? reinterpret_cast<const Model *>(mp)->sin : nullptr; }

int lbk_model_get_config(const lbk_model *mp, lbk_model_config *out) {
    if (!mp || !out) return fail(LBK_ERR_INVALID, "lbk_model_get_config: null argument");
    *out = reinterpret_cast<const Model *>(mp)->cfg;
    return LBK_OK;
}

int lbk_kv_cache_free(lbk_kv_cache *cp) {
    if (!cp) return LBK_OK;
    Cache *c = reinterpret_cast<Cache *>(cp);
    cudaSetDevice(c->model->ctx->device);
    cudaDeviceSynchronize();
    if (c->step) cudaGraphExecDestroy(c->step);
    for (void *p : c->device_allocs) cudaFree(p);
    for (void *p : c->pf_allocs) cudaFree(p);
    delete c;
    return LBK_OK;
}

int lbk_model_new_cache(lbk_model *mp, size_t batch, size_t capacity, lbk_kv_cache **out) {
    if (!mp || !out) return fail(LBK_ERR_INVALID, "lbk_model_new_cache: null argument");
    *out = nullptr;
    Model *m = reinterpret_cast<Model *>(mp);
    if (m->world > 1)
        return fail(LBK_ERR_UNSUPPORTED, "this model holds shard %d of %d: its step needs the other ranks (drive it through the tensor-parallel layer calls)", m->rank, m->world);
    if (batch == 0 || batch > LBK_GEMV_MAX_M) return fail(LBK_ERR_UNSUPPORTED, "a cache serves 1..%d sequences (got %zu)", LBK_GEMV_MAX_M, batch);
    if (capacity == 0) capacity = m->cfg.max_position_embeddings;
    if (capacity > m->cfg.max_position_embeddings) return fail(LBK_ERR_INVALID, "capacity %zu exceeds max_position_embeddings %zu", capacity, m->cfg.max_position_embeddings);
    LBK_CUDA(cudaSetDevice(m->ctx->device));
    std::unique_ptr<Cache, int (*)(Cache *)> cache(new Cache(), [](Cache *c) { return lbk_kv_cache_free(reinterpret_cast<lbk_kv_cache *>(c)); });
    Cache *c = cache.get();
    c->model = m;
    c->b = batch;
    c->cap = capacity;
    const lbk_model_config &cfg = m->cfg;
    const size_t H = cfg.hidden_size, I = cfg.intermediate_size, nh = cfg.num_attention_heads, kvh = cfg.num_key_value_heads, hd = m->head_dim;
    c->splits = std::min<size_t>((capacity + 31) / 32, 256);  // 32 positions per attention slice (the Python mirror's attention_splits)
    const size_t kv_elems = cfg.num_hidden_layers * batch * kvh * capacity * hd;
    LBK_TRY(dev_alloc(c->device_allocs, kv_elems * 2, reinterpret_cast<void **>(&c->k)));
    LBK_TRY(dev_alloc(c->device_allocs, kv_elems * 2, reinterpret_cast<void **>(&c->v)));
    LBK_CUDA(cudaMemset(c->k, 0, kv_elems * 2));
    LBK_CUDA(cudaMemset(c->v, 0, kv_elems * 2));
    struct { void **p; size_t bytes; } bufs[] = {
        {reinterpret_cast<void **>(&c->pos), batch * 4}, {reinterpret_cast<void **>(&c->active), batch * 4}, {reinterpret_cast<void **>(&c->tokens), batch * 4}, {reinterpret_cast<void **>(&c->next), batch * 4},
        {reinterpret_cast<void **>(&c->counters), batch * kvh * 4}, {reinterpret_cast<void **>(&c->x), batch * H * 4},
        {reinterpret_cast<void **>(&c->x2), batch * H * 4}, {reinterpret_cast<void **>(&c->n), batch * H * 4},
        {reinterpret_cast<void **>(&c->q), batch * nh * hd * 4}, {reinterpret_cast<void **>(&c->kk), batch * kvh * hd * 4},
        {reinterpret_cast<void **>(&c->vv), batch * kvh * hd * 4}, {reinterpret_cast<void **>(&c->attn), batch * nh * hd * 4},
        {reinterpret_cast<void **>(&c->o), batch * H * 4}, {reinterpret_cast<void **>(&c->g), batch * I * 4}, {reinterpret_cast<void **>(&c->u), batch * I * 4},
        {reinterpret_cast<void **>(&c->d), batch * H * 4}, {reinterpret_cast<void **>(&c->act), batch * I * 4},
        {reinterpret_cast<void **>(&c->q8), batch * ((std::max(std::max(H, I), nh * hd) + 127) / 128 * 128)},
        {reinterpret_cast<void **>(&c->qscale), batch * 4}, {reinterpret_cast<void **>(&c->qsum), batch * 4},
        {reinterpret_cast<void **>(&c->logits), batch * cfg.vocab_size * 4}, {reinterpret_cast<void **>(&c->scratch), batch * nh * c->splits * (hd + 4) * 4}};
    for (auto &bf : bufs) {
        LBK_TRY(dev_alloc(c->device_allocs, bf.bytes, bf.p));
        LBK_CUDA(cudaMemset(*bf.p, 0, bf.bytes));
    }
    c->lens.assign(batch, 0);
    const std::vector<int32_t> ones(batch, 1);
    LBK_CUDA(cudaMemcpy(c->active, ones.data(), batch * 4, cudaMemcpyHostToDevice));
    *out = reinterpret_cast<lbk_kv_cache *>(cache.release());
    return LBK_OK;
}

size_t lbk_kv_cache_len(const lbk_kv_cache *cp) { return cp ? reinterpret_cast<const Cache *>(cp)->lens[0] : 0; }

int lbk_kv_cache_reset(lbk_kv_cache *cp) {
    if (!cp) return fail(LBK_ERR_INVALID, "cache is null");
    Cache *c = reinterpret_cast<Cache *>(cp);
    LBK_CUDA(cudaSetDevice(c->model->ctx->device));
    LBK_CUDA(cudaDeviceSynchronize());
    LBK_CUDA(cudaMemset(c->pos, 0, c->b * 4));
    c->lens.assign(c->b, 0);
    return LBK_OK;
}

int lbk_model_decode(lbk_model *mp, lbk_kv_cache *cp, const int32_t *tokens_dev, float *logits_dev, int32_t *next_dev, void *stream) {
    if (!mp || !cp || !tokens_dev) return fail(LBK_ERR_INVALID, "lbk_model_decode: null argument");
    Model *m = reinterpret_cast<Model *>(mp);
    Cache *c = reinterpret_cast<Cache *>(cp);
    if (c->model != m) return fail(LBK_ERR_INVALID, "the cache belongs to another model");
    for (size_t l : c->lens)
        if (l >= c->cap) return fail(LBK_ERR_INVALID, "the cache is full (%zu positions)", c->cap);
    LBK_CUDA(cudaSetDevice(m->ctx->device));
    LBK_TRY(ensure_graph(m, c));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LBK_CUDA(cudaMemcpyAsync(c->tokens, tokens_dev, c->b * 4, cudaMemcpyDeviceToDevice, st));
    LBK_CUDA(cudaGraphLaunch(c->step, st));
    m->ctx->launches += 7 * m->cfg.num_hidden_layers + 6;
    if (logits_dev) LBK_CUDA(cudaMemcpyAsync(logits_dev, c->logits, c->b * m->cfg.vocab_size * 4, cudaMemcpyDeviceToDevice, st));
    if (next_dev) LBK_CUDA(cudaMemcpyAsync(next_dev, c->next, c->b * 4, cudaMemcpyDeviceToDevice, st));
    for (size_t &l : c->lens) l += 1;
    return LBK_OK;
}

int lbk_model_forward(lbk_model *mp, lbk_kv_cache *cp, const uint32_t *tokens, size_t n, int all_logits, float *logits_out) {
    if (!mp || !cp || (n && !tokens)) return fail(LBK_ERR_INVALID, "lbk_model_forward: null argument");
    Model *m = reinterpret_cast<Model *>(mp);
    Cache *c = reinterpret_cast<Cache *>(cp);
    if (c->model != m) return fail(LBK_ERR_INVALID, "the cache belongs to another model");
    if (c->b != 1) return fail(LBK_ERR_INVALID, "lbk_model_forward drives one sequence; this cache was made for %zu", c->b);
    if (n == 0) return LBK_OK;
    if (c->lens[0] + n > c->cap) return fail(LBK_ERR_INVALID, "%zu tokens do not fit: %zu of %zu positions are used", n, c->lens[0], c->cap);
    LBK_CUDA(cudaSetDevice(m->ctx->device));
    cudaStream_t st = m->ctx->own_stream;
    const size_t V = m->cfg.vocab_size;
    for (size_t i = 0; i < n; ++i)
        if (tokens[i] >= V) return fail(LBK_ERR_INVALID, "token %u is outside the vocabulary of %zu", tokens[i], V);
    if (n >= 2) {  // a prompt: whole chunks of rows through the projections at once
        for (size_t i0 = 0; i0 < n; i0 += m->prefill_rows) {
            const size_t rows = n - i0 < m->prefill_rows ? n - i0 : m->prefill_rows;
            const bool last = i0 + rows == n;
            float *dst = logits_out ? (all_logits ? logits_out + i0 * V : (last ? logits_out : nullptr)) : nullptr;
            if (rows == 1) {  // a single left-over token takes the decode step
                LBK_TRY(lbk_model_forward(mp, cp, tokens + i0, 1, all_logits, dst));
            } else {
                LBK_TRY(prefill_chunk(m, c, 0, tokens + i0, rows, all_logits, dst));
            }
        }
        return LBK_OK;
    }
    LBK_TRY(ensure_graph(m, c));
    {
        const int32_t tk = static_cast<int32_t>(tokens[0]);
        LBK_CUDA(cudaMemcpyAsync(c->tokens, &tk, 4, cudaMemcpyHostToDevice, st));
        LBK_CUDA(cudaStreamSynchronize(st));  // `tk` is a stack variable
        LBK_CUDA(cudaGraphLaunch(c->step, st));
        m->ctx->launches += 7 * m->cfg.num_hidden_layers + 6;
        c->lens[0] += 1;
        if (logits_out) LBK_CUDA(cudaMemcpyAsync(logits_out, c->logits, V * 4, cudaMemcpyDeviceToHost, st));
    }
    LBK_CUDA(cudaStreamSynchronize(st));
    return LBK_OK;
}

int lbk_model_set_prefill_rows(lbk_model *mp, size_t rows) {
    if (!mp) return fail(LBK_ERR_INVALID, "lbk_model_set_prefill_rows: model is null");
    if (rows < 1 || rows > 8192) return fail(LBK_ERR_INVALID, "rows per prompt pass must be 1..8192 (got %zu)", rows);
    reinterpret_cast<Model *>(mp)->prefill_rows = rows;
    return LBK_OK;
}

size_t lbk_kv_cache_len_seq(const lbk_kv_cache *cp, size_t seq) {
    const Cache *c = reinterpret_cast<const Cache *>(cp);
    return c && seq < c->b ? c->lens[seq] : 0;
}

int lbk_batcher_create(lbk_model *mp, size_t slots, size_t capacity, lbk_batcher **out) {
    if (!mp || !out) return fail(LBK_ERR_INVALID, "lbk_batcher_create: null argument");
    *out = nullptr;
    lbk_kv_cache *cache = nullptr;
    LBK_TRY(lbk_model_new_cache(mp, slots, capacity, &cache));
    Batcher *b = new Batcher();
    b->model = reinterpret_cast<Model *>(mp);
    b->cache = reinterpret_cast<Cache *>(cache);
    b->slot_req.assign(slots, 0);
    *out = reinterpret_cast<lbk_batcher *>(b);
    return LBK_OK;
}

int lbk_batcher_destroy(lbk_batcher *bp) {
    if (!bp) return LBK_OK;
    Batcher *b = reinterpret_cast<Batcher *>(bp);
    lbk_kv_cache_free(reinterpret_cast<lbk_kv_cache *>(b->cache));
    delete b;
    return LBK_OK;
}

int lbk_batcher_submit(lbk_batcher *bp, const uint32_t *prompt, size_t n, size_t max_new_tokens, int32_t eos_token, uint64_t *id_out) {
    if (!bp || !prompt || !id_out) return fail(LBK_ERR_INVALID, "lbk_batcher_submit: null argument");
    Batcher *b = reinterpret_cast<Batcher *>(bp);
    if (n == 0 || max_new_tokens == 0) return fail(LBK_ERR_INVALID, "a request needs a prompt and at least one token to generate");
    if (n > b->cache->cap) return fail(LBK_ERR_INVALID, "a prompt of %zu tokens does not fit %zu positions", n, b->cache->cap);
    const size_t V = b->model->cfg.vocab_size;
    for (size_t i = 0; i < n; ++i)
        if (prompt[i] >= V) return fail(LBK_ERR_INVALID, "token %u is outside the vocabulary of %zu", prompt[i], V);
    Request r;
    r.id = b->next_id++;
    r.prompt.assign(prompt, prompt + n);
    r.max_new = max_new_tokens;
    r.eos = eos_token;
    b->queue.push_back(r.id);
    *id_out = r.id;
    b->reqs.emplace(r.id, std::move(r));
    return LBK_OK;
}

int lbk_batcher_step(lbk_batcher *bp, size_t *pending_out) {
    if (!bp) return fail(LBK_ERR_INVALID, "lbk_batcher_step: null argument");
    Batcher *b = reinterpret_cast<Batcher *>(bp);
    Model *m = b->model;
    Cache *c = b->cache;
    LBK_CUDA(cudaSetDevice(m->ctx->device));
    cudaStream_t st = m->ctx->own_stream;
    const size_t slots = c->b;
    // a sequence is finished by its end token, its budget, or a full cache; its slot goes back at once
    auto finished = [&](const Request &r, size_t slot) {
        return (r.eos >= 0 && static_cast<int32_t>(r.out.back()) == r.eos) || r.out.size() >= r.max_new || c->lens[slot] >= c->cap;
    };
    auto retire = [&](Request &r, size_t slot) -> int {
        r.done = true;
        r.slot = -1;
        b->slot_req[slot] = 0;
        const int32_t zero = 0;  // an idle slot still runs through the step: keep its position inside the cache
        LBK_CUDA(cudaMemcpy(c->pos + slot, &zero, 4, cudaMemcpyHostToDevice));
        c->lens[slot] = 0;
        return LBK_OK;
    };
    // admission: prompts into free slots
    for (size_t slot = 0; slot < slots && !b->queue.empty(); ++slot) {
        if (b->slot_req[slot]) continue;
        Request &r = b->reqs.at(b->queue.front());
        b->queue.pop_front();
        int32_t first = 0;
        for (size_t i0 = 0; i0 < r.prompt.size(); i0 += m->prefill_rows) {
            const size_t rows = std::min(m->prefill_rows, r.prompt.size() - i0);
            const bool last = i0 + rows == r.prompt.size();
            LBK_TRY(prefill_chunk(m, c, slot, r.prompt.data() + i0, rows, 0, nullptr, last ? &first : nullptr));
        }
        r.out.push_back(static_cast<uint32_t>(first));
        r.slot = static_cast<int>(slot);
        b->slot_req[slot] = r.id;
        if (finished(r, slot)) LBK_TRY(retire(r, slot));
    }
    // one decode step for the occupied slots
    std::vector<int32_t> tokens(slots, 0), active(slots, 0), next(slots, 0);
    size_t n_active = 0;
    for (size_t slot = 0; slot < slots; ++slot)
        if (b->slot_req[slot]) {
            tokens[slot] = static_cast<int32_t>(b->reqs.at(b->slot_req[slot]).out.back());
            active[slot] = 1;
            ++n_active;
        }
    if (n_active) {
        LBK_TRY(ensure_graph(m, c));
        LBK_CUDA(cudaMemcpyAsync(c->tokens, tokens.data(), slots * 4, cudaMemcpyHostToDevice, st));
        LBK_CUDA(cudaMemcpyAsync(c->active, active.data(), slots * 4, cudaMemcpyHostToDevice, st));
        LBK_CUDA(cudaStreamSynchronize(st));  // the host vectors are pageable
        LBK_CUDA(cudaGraphLaunch(c->step, st));
        m->ctx->launches += 7 * m->cfg.num_hidden_layers + 6;
        LBK_CUDA(cudaMemcpyAsync(next.data(), c->next, slots * 4, cudaMemcpyDeviceToHost, st));
        LBK_CUDA(cudaStreamSynchronize(st));
        for (size_t slot = 0; slot < slots; ++slot) {
            if (!b->slot_req[slot]) continue;
            Request &r = b->reqs.at(b->slot_req[slot]);
            c->lens[slot] += 1;
            r.out.push_back(static_cast<uint32_t>(next[slot]));
            if (finished(r, slot)) LBK_TRY(retire(r, slot));
        }
    }
    if (pending_out) {
        size_t occupied = 0;
        for (uint64_t id : b->slot_req) occupied += id != 0;
        *pending_out = occupied + b->queue.size();
    }
    return LBK_OK;
}

int lbk_batcher_poll(lbk_batcher *bp, uint64_t id, uint32_t *tokens_out, size_t capacity, size_t *n_out, int *done_out) {
    if (!bp || !n_out) return fail(LBK_ERR_INVALID, "lbk_batcher_poll: null argument");
    Batcher *b = reinterpret_cast<Batcher *>(bp);
    auto it = b->reqs.find(id);
    if (it == b->reqs.end()) return fail(LBK_ERR_INVALID, "no request %llu", static_cast<unsigned long long>(id));
    const Request &r = it->second;
    *n_out = r.out.size();
    if (tokens_out)
        for (size_t i = 0; i < r.out.size() && i < capacity; ++i) tokens_out[i] = r.out[i];
    if (done_out) *done_out = r.done ? 1 : 0;
    return LBK_OK;
}

int lbk_batcher_forget(lbk_batcher *bp, uint64_t id) {
    if (!bp) return fail(LBK_ERR_INVALID, "lbk_batcher_forget: null argument");
    Batcher *b = reinterpret_cast<Batcher *>(bp);
    auto it = b->reqs.find(id);
    if (it == b->reqs.end()) return fail(LBK_ERR_INVALID, "no request %llu", static_cast<unsigned long long>(id));
    if (!it->second.done) return fail(LBK_ERR_INVALID, "request %llu is still running", static_cast<unsigned long long>(id));
    b->reqs.erase(it);
    return LBK_OK;
}

}  // extern "C"
