// Quantisation-table ingestion: turns a float graph plus an `odla_value_quant_info[]` table
// (ODLA/include/ODLA/ops/odla_ops_quantization.h:33-41 in the reference; written by
// utils/halo_pgq.py:309-327 as one record per value with ch_idx = -channels followed by one
// record per channel, and declared by generated code, lib/target/generic_cpp/generic_cxx_codegen.cc:110-116)
// into the Quantize / Dequantize form the planner already runs on the int8 tensor cores.
//
// The reference defines the table but none of its platforms consumes it, so the meaning given to a
// record here is this library's own: symmetric int8, scale = max(|min|, |max|) / 127 (a record whose
// min and max are both zero but whose scale is positive supplies the scale directly); weights use
// their per-channel records when the table has them for every output channel, else the ranges of the
// constant itself.  For every convolution (channels-last, one group) and rank-2 Gemm whose data
// operand has a record and whose weights are a float constant, the rewrite inserts
//     x -> Quantize(s_x) -> Dequantize(s_x) -> op      and      W -> Dequantize(int8 W_q, s_w[k]) -> op
// (and, for weights the compiler already quantised to asymmetric uint8, W_u -> Dequantize(W_u, s_w, zp_w) -> op),
// which is exactly what a hand-written QDQ model holds; everything downstream (operand absorption,
// requantising epilogues, bit-exact int32 accumulation) is the planner's existing int8 path.
#include <cmath>
#include <cstring>

#include "common.h"

namespace b200 {

namespace {

struct Range {
  float mn = 0.f, mx = 0.f, scale = 0.f, offset = 0.f;
  bool have = false;
  std::vector<std::pair<float, float>> ch;  // per-channel (min, max)
  std::vector<bool> ch_have;
};

float symmetric_scale(float mn, float mx, float given) {
  float a = std::fmax(std::fabs(mn), std::fabs(mx));
  if (a == 0.f && given > 0.f) return given;
  if (a == 0.f) return 1.f;
  return a / 127.f;
}

}  // namespace

odla_status apply_quant_table(_odla_computation* c) {
  if (c->quant_applied || c->quant_table.empty()) return ODLA_SUCCESS;
  c->quant_applied = true;
  std::map<std::string, Range> table;
  for (const auto& rec : c->quant_table) {
    const char* id = (const char*)rec.value_id;
    if (!id) continue;
    Range& r = table[id];
    if (rec.ch_idx < 0) {
      r.have = true;
      r.mn = rec.min; r.mx = rec.max; r.scale = rec.scale; r.offset = rec.offset;
    } else {
      if ((size_t)rec.ch_idx >= r.ch.size()) { r.ch.resize((size_t)rec.ch_idx + 1); r.ch_have.resize((size_t)rec.ch_idx + 1, false); }
      r.ch[(size_t)rec.ch_idx] = {rec.min, rec.max};
      r.ch_have[(size_t)rec.ch_idx] = true;
    }
  }
  auto own = [&](const void* data, size_t bytes) -> const void* {
    c->owned_consts.emplace_back(new std::vector<uint8_t>((const uint8_t*)data, (const uint8_t*)data + bytes));
    return c->owned_consts.back()->data();
  };
  std::vector<std::unique_ptr<_odla_value>> out;
  out.reserve(c->nodes.size() + 8);
  auto make = [&](const std::string& name, OpKind kind, odla_element_type et, const odla_value_shape& shape, std::vector<odla_value> in,
                  std::vector<int64_t> ia) -> odla_value {
    auto v = std::make_unique<_odla_value>();
    v->name = name;
    v->type.element_type = et;
    v->type.shape = shape;
    v->kind = kind;
    v->in = std::move(in);
    v->ia = std::move(ia);
    odla_value r = v.get();
    out.push_back(std::move(v));
    return r;
  };
  auto scalar_const = [&](const std::string& name, float s) {
    odla_value_shape sh{};
    sh.size = 1; sh.dims[0] = 1;
    odla_value v = make(name, OP_CONST, ODLA_FLOAT32, sh, {}, {});
    v->host = own(&s, sizeof(float));
    return v;
  };
  std::map<odla_value, odla_value> dq_of;  // one Quantize/Dequantize pair per quantised activation
  int rewritten = 0;
  for (auto& up : c->nodes) {
    _odla_value* v = up.get();
    bool conv = v->kind == OP_CONV && v->ia.size() >= 2 && v->ia[0] == 1 && v->ia[1] == 1;
    bool gemm = v->kind == OP_GEMM && v->type.shape.size == 2 && v->ia.size() >= 2 && v->ia[0] == 0;
    odla_value x = (conv || gemm) ? v->in[0] : nullptr, w = (conv || gemm) ? v->in[1] : nullptr;
    auto xr = x ? table.find(x->name) : table.end();
    // ---- weights already quantised by the compiler: -quantize-weights=quint8 turns every float constant into uint8
    // with one scale and one zero point (lib/quantizer/weights_quantizer.cc:84-182: q = clamp(round(w / scale + zp), 0,
    // 255)) and the bias of a convolution / Gemm into int32 with scale s_in * s_w (:139-172); the table carries those
    // scales.  The filter becomes Dequantize(uint8, scale, zp), the bias a float constant b_q * (s_in * s_w).
    auto wr8 = w ? table.find(w->name) : table.end();
    if ((conv || gemm) && x && w && !v->poison && x->kind != OP_CONST && is_float_type(x->type.element_type) && w->kind == OP_CONST &&
        (w->type.element_type == ODLA_UINT8 || w->type.element_type == ODLA_QUINT8) && w->host && xr != table.end() && xr->second.have &&
        wr8 != table.end() && wr8->second.have && wr8->second.scale > 0.f) {
      odla_value xdq;
      auto hit = dq_of.find(x);
      if (hit != dq_of.end()) xdq = hit->second;
      else {
        float sx = symmetric_scale(xr->second.mn, xr->second.mx, xr->second.scale);
        odla_value sc = scalar_const(x->name + "_qt_scale", sx);
        int64_t last = x->type.shape.size - 1;
        odla_value q = make(x->name + "_qt_q", OP_QUANTIZE, ODLA_INT8, x->type.shape, {x, sc, nullptr}, {last});
        xdq = make(x->name + "_qt_dq", OP_DEQUANTIZE, x->type.element_type, x->type.shape, {q, sc, nullptr}, {last});
        dq_of[x] = xdq;
      }
      odla_value wsc = scalar_const(w->name + "_qt_scale", wr8->second.scale);
      odla_value_shape one{};
      one.size = 1; one.dims[0] = 1;
      odla_value wzp = make(w->name + "_qt_zp", OP_CONST, ODLA_INT32, one, {}, {});
      const int32_t zp = (int32_t)std::nearbyintf(wr8->second.offset);
      wzp->host = own(&zp, sizeof(zp));
      odla_value wdq = make(w->name + "_qt_dq", OP_DEQUANTIZE, ODLA_FLOAT32, w->type.shape, {w, wsc, wzp}, {0});
      v->in[0] = xdq;
      v->in[1] = wdq;
      odla_value b = v->in.size() > 2 ? v->in[2] : nullptr;
      if (b && b->kind == OP_CONST && (b->type.element_type == ODLA_INT32 || b->type.element_type == ODLA_QINT32) && b->host) {
        // the scales the compiler divided the bias by are the table's own records of the two operands
        const float sb = xr->second.scale * wr8->second.scale;
        const int64_t nb = numel(b->type.shape);
        std::vector<float> bf((size_t)nb);
        for (int64_t i = 0; i < nb; ++i) bf[(size_t)i] = (float)((const int32_t*)b->host)[i] * sb;
        odla_value bc = make(b->name + "_qt_f", OP_CONST, ODLA_FLOAT32, b->type.shape, {}, {});
        bc->host = own(bf.data(), bf.size() * sizeof(float));
        v->in[2] = bc;
      }
      ++rewritten;
      out.push_back(std::move(up));
      continue;
    }
    if ((conv || gemm) && x && w && !v->poison && x->kind != OP_CONST && is_float_type(x->type.element_type) && w->kind == OP_CONST &&
        w->type.element_type == ODLA_FLOAT32 && w->host && xr != table.end() && xr->second.have) {
      // ---- activation ----
      odla_value xdq;
      auto hit = dq_of.find(x);
      if (hit != dq_of.end()) xdq = hit->second;
      else {
        float sx = symmetric_scale(xr->second.mn, xr->second.mx, xr->second.scale);
        odla_value sc = scalar_const(x->name + "_qt_scale", sx);
        int64_t last = x->type.shape.size - 1;
        odla_value q = make(x->name + "_qt_q", OP_QUANTIZE, ODLA_INT8, x->type.shape, {x, sc, nullptr}, {last});
        xdq = make(x->name + "_qt_dq", OP_DEQUANTIZE, x->type.element_type, x->type.shape, {q, sc, nullptr}, {last});
        dq_of[x] = xdq;
      }
      // ---- weights: output channels are the last axis of an HWIO kernel and of a [K, N] matrix, the first of a transposed one ----
      const auto& ws = w->type.shape;
      const int64_t n = numel(ws);
      const bool k_first = gemm && v->ia[1] != 0;
      const int64_t K = k_first ? ws.dims[0] : ws.dims[ws.size - 1];
      const float* wf = (const float*)w->host;
      auto idx = [&](int64_t k, int64_t j) { return k_first ? k * (n / K) + j : j * K + k; };
      std::vector<float> s_w((size_t)K);
      auto wr = table.find(w->name);
      bool from_table = wr != table.end() && (int64_t)wr->second.ch.size() == K;
      if (from_table)
        for (int64_t k = 0; k < K; ++k) from_table = from_table && wr->second.ch_have[(size_t)k];
      for (int64_t k = 0; k < K; ++k) {
        float mn = 0.f, mx = 0.f;
        if (from_table) { mn = wr->second.ch[(size_t)k].first; mx = wr->second.ch[(size_t)k].second; }
        else
          for (int64_t j = 0; j < n / K; ++j) { float t = wf[idx(k, j)]; mn = std::fmin(mn, t); mx = std::fmax(mx, t); }
        s_w[(size_t)k] = symmetric_scale(mn, mx, 0.f);
      }
      std::vector<int8_t> wq((size_t)n);
      for (int64_t k = 0; k < K; ++k)
        for (int64_t j = 0; j < n / K; ++j) {
          float t = std::nearbyintf(wf[idx(k, j)] / s_w[(size_t)k]);  // round to nearest even, like the Quantize operator
          t = std::fmin(std::fmax(t, -127.f), 127.f);
          wq[(size_t)idx(k, j)] = (int8_t)t;
        }
      odla_value wqc = make(w->name + "_qt_q", OP_CONST, ODLA_INT8, ws, {}, {});
      wqc->host = own(wq.data(), wq.size());
      odla_value_shape ss{};
      ss.size = 1; ss.dims[0] = K;
      odla_value wsc = make(w->name + "_qt_scale", OP_CONST, ODLA_FLOAT32, ss, {}, {});
      wsc->host = own(s_w.data(), s_w.size() * sizeof(float));
      odla_value wdq = make(w->name + "_qt_dq", OP_DEQUANTIZE, ODLA_FLOAT32, ws, {wqc, wsc, nullptr}, {k_first ? 0 : (int64_t)ws.size - 1});
      v->in[0] = xdq;
      v->in[1] = wdq;
      ++rewritten;
    }
    out.push_back(std::move(up));
  }
  c->nodes = std::move(out);
  for (size_t i = 0; i < c->nodes.size(); ++i) {
    c->nodes[i]->index = (int)i;
    c->by_name[c->nodes[i]->name] = c->nodes[i].get();
  }
  B2_INFO("quantisation table: %d records, %d convolutions / Gemms now run in int8", (int)c->quant_table.size(), rewritten);
  return ODLA_SUCCESS;
}

}  // namespace b200
