// Runs the reference's own Qwen3Model::forward (pulsar-core/src/model/qwen3.cpp,
// paged_forward.cpp, runtime/kv/active_buffer.cpp, compiled unchanged) on the CPU for one
// whole prompt and writes the logits of every position.
//
// The reference's five CUDA-only ops are supplied here as plain ATen restatements of their
// contracts (pulsar-core/inc/pulsar/ops.hpp): what this anchors is the model code's order of
// operations, norm placement, residuals, head tying and the paged bookkeeping; the
// arithmetic inside norm, rope and attention below rests on the formulas.  Keys are rotated
// once (before write_kv, as paged_forward.cpp:23-26 does) and not again on read.
//
// Input file (little endian): int32 L, Hq, Hkv, D, hidden, inter, V, untied, page, T;
// float64 theta, eps; int32 tokens[T]; then float32 tensors in this order: embed, norm,
// per layer: input_layernorm, post_attention_layernorm, q, k, v, o, q_norm, k_norm, gate, up,
// down; then lm_head if untied.  Output: float32 logits [T, V].
#include "pulsar/model/qwen3.hpp"
#include "pulsar/ops.hpp"
#include "pulsar/rope.hpp"
#include "pulsar/runtime/kv/active_buffer.hpp"

#include <ATen/ATen.h>

#include <cstdio>
#include <fstream>
#include <iostream>
#include <vector>

namespace pulsar {

at::Tensor rmsnorm_cuda(const at::Tensor& x, const at::Tensor& w, double eps) {
    auto xf = x.to(at::kFloat);
    auto inv = at::rsqrt(xf.pow(2).mean(-1, true) + static_cast<float>(eps));
    return (xf * inv * w.to(at::kFloat)).to(x.scalar_type());
}

at::Tensor rope_cuda(const at::Tensor& x, const at::Tensor& pos, double theta) {   // x [H, S, D]
    return rope_rotate(x.to(at::kFloat), pos.view({1, -1}), theta).to(x.scalar_type());
}

void write_kv_cuda(const at::Tensor& kp, const at::Tensor& vp, const at::Tensor& k, const at::Tensor& v,
                   const at::Tensor& slots) {
    auto fk = kp.view({-1, kp.size(2), kp.size(3)});
    auto fv = vp.view({-1, vp.size(2), vp.size(3)});
    fk.index_copy_(0, slots.to(at::kLong), k);
    fv.index_copy_(0, slots.to(at::kLong), v);
}

void reposition_kv_cuda(const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&, double) {
    TORCH_CHECK(false, "not used");
}

static at::Tensor attend(const at::Tensor& q, const at::Tensor& kp, const at::Tensor& vp, const at::Tensor& tables,
                         const at::Tensor& cu, const at::Tensor& lens, double scale) {
    const int64_t S = lens.size(0), H = q.size(1), D = q.size(2), KV = kp.size(2), ps = kp.size(1), group = H / KV;
    auto out = at::zeros_like(q, at::kFloat);
    for (int64_t s = 0; s < S; ++s) {
        const int64_t ctx = lens[s].item<int64_t>();
        const int64_t q0 = cu.defined() ? cu[s].item<int64_t>() : s;
        const int64_t q1 = cu.defined() ? cu[s + 1].item<int64_t>() : s + 1;
        auto pages = tables[s].slice(0, 0, (ctx + ps - 1) / ps).to(at::kLong);
        auto k = kp.index_select(0, pages).view({-1, KV, D}).slice(0, 0, ctx).to(at::kFloat);
        auto v = vp.index_select(0, pages).view({-1, KV, D}).slice(0, 0, ctx).to(at::kFloat);
        for (int64_t t = q0; t < q1; ++t) {
            const int64_t p = ctx - (q1 - q0) + (t - q0);
            for (int64_t h = 0; h < H; ++h) {
                auto scores = at::mv(k.select(1, h / group).slice(0, 0, p + 1), q[t][h].to(at::kFloat)) * scale;
                out[t][h] = at::mv(v.select(1, h / group).slice(0, 0, p + 1).t(), at::softmax(scores, 0));
            }
        }
    }
    return out.to(q.scalar_type());
}

at::Tensor attn_prefill_cuda(const at::Tensor& q, const at::Tensor& kp, const at::Tensor& vp, const at::Tensor& pt,
                             const at::Tensor& cu, const at::Tensor& sk, const at::Tensor&, double, double scale,
                             const std::optional<at::Tensor>&, const std::optional<at::Tensor>&,
                             const std::optional<at::Tensor>&, double, const std::optional<at::Tensor>&) {
    return attend(q, kp, vp, pt, cu, sk, scale);
}

at::Tensor attn_decode_cuda(const at::Tensor& q, const at::Tensor& kp, const at::Tensor& vp, const at::Tensor& pt,
                            const at::Tensor& cl, const at::Tensor&, double, double scale,
                            const std::optional<at::Tensor>&, const std::optional<at::Tensor>&,
                            const std::optional<at::Tensor>&, double, const std::optional<at::Tensor>&, int64_t) {
    return attend(q, kp, vp, pt, {}, cl, scale);
}

}  // namespace pulsar

using namespace pulsar;

int main(int argc, char** argv) {
    if (argc != 3) { std::cerr << "usage: golden_ref INPUT OUTPUT\n"; return 2; }
    std::ifstream in(argv[1], std::ios::binary);
    int32_t hdr[10];
    in.read(reinterpret_cast<char*>(hdr), sizeof hdr);
    const int64_t L = hdr[0], H = hdr[1], KV = hdr[2], D = hdr[3], hid = hdr[4], inter = hdr[5], V = hdr[6];
    const bool untied = hdr[7] != 0;
    const int64_t page = hdr[8], T = hdr[9];
    double consts[2];
    in.read(reinterpret_cast<char*>(consts), sizeof consts);
    std::vector<int32_t> ids(T);
    in.read(reinterpret_cast<char*>(ids.data()), T * 4);
    auto read = [&](std::initializer_list<int64_t> shape) {
        auto t = at::empty(shape, at::kFloat);
        in.read(reinterpret_cast<char*>(t.data_ptr<float>()), t.numel() * 4);
        return t;
    };
    c10::Dict<std::string, at::Tensor> w;
    w.insert("model.embed_tokens.weight", read({V, hid}));
    w.insert("model.norm.weight", read({hid}));
    for (int64_t i = 0; i < L; ++i) {
        const std::string p = "model.layers." + std::to_string(i) + ".";
        w.insert(p + "input_layernorm.weight", read({hid}));
        w.insert(p + "post_attention_layernorm.weight", read({hid}));
        w.insert(p + "self_attn.q_proj.weight", read({H * D, hid}));
        w.insert(p + "self_attn.k_proj.weight", read({KV * D, hid}));
        w.insert(p + "self_attn.v_proj.weight", read({KV * D, hid}));
        w.insert(p + "self_attn.o_proj.weight", read({hid, H * D}));
        w.insert(p + "self_attn.q_norm.weight", read({D}));
        w.insert(p + "self_attn.k_norm.weight", read({D}));
        w.insert(p + "mlp.gate_proj.weight", read({inter, hid}));
        w.insert(p + "mlp.up_proj.weight", read({inter, hid}));
        w.insert(p + "mlp.down_proj.weight", read({hid, inter}));
    }
    if (untied) w.insert("lm_head.weight", read({V, hid}));
    TORCH_CHECK(in.good(), "input file too short");

    Qwen3Model model(L, H, KV, D, hid, inter, V, consts[0], consts[1], w);
    ActiveBuffer kv(L, (T + page - 1) / page + 1, page, KV, H, D, at::kFloat, "cpu", consts[0]);
    kv.allocate(0, T);
    GroupBatch g;
    g.tokens = at::tensor(std::vector<int64_t>(ids.begin(), ids.end()), at::kLong);
    g.pos = at::arange(T);
    g.slot_mapping = kv.slot_mapping(0, 0, T);
    g.page_tables = kv.page_table(0).view({1, -1});
    g.cu_seqlens_q = at::tensor({0, static_cast<int>(T)}, at::kInt);
    g.seqlens_k = at::tensor({static_cast<int>(T)}, at::kInt);
    StepBatch batch;
    batch.prefill = g;
    auto logits = model.forward(batch, kv).prefill->to(at::kFloat).contiguous();
    TORCH_CHECK(logits.size(0) == T && logits.size(1) == V, "unexpected logits shape");
    std::ofstream out(argv[2], std::ios::binary);
    out.write(reinterpret_cast<const char*>(logits.data_ptr<float>()), logits.numel() * 4);
    std::cout << "wrote " << T << " x " << V << " logits\n";
    return 0;
}
