// odla_StoreExecutable / odla_LoadExecutable: a computation as one self-contained file.
//
// What the reference's TensorRT platform stores is a serialised engine -- the whole model, weights included
// (ODLA/platforms/tensorrt/odla_tensorrt.cc:537-559) -- and what it loads becomes a new current computation whose
// arguments and outputs are found by name (odla_tensorrt.cc:703-811).  The same contract here: the file holds the
// recorded graph (every node with its type, operands and attributes), the constants' bytes, the computation's items
// (storage type, GPU count, sub-batches, quantisation table) and the prepared constants -- filters already converted
// to the storage type and repacked K-major for the tensor-core kernel, which is the expensive part of planning.  What
// is NOT stored is anything that contains a device address (arenas, tensor maps, captured CUDA graphs): those are
// rebuilt by the first execute on whatever GPUs the loading process sees.
//
// Layout (little endian): "ODLAB200" magic, u32 version, u64 FNV-1a hash of everything after the header, then the
// sections in the order written by Writer below.  A file whose hash or version does not match is refused.
#include <cstdio>
#include <cstring>
#include <fstream>

#include "common.h"

using namespace b200;

namespace {

constexpr char kMagic[8] = {'O', 'D', 'L', 'A', 'B', '2', '0', '0'};
constexpr uint32_t kVersion = 1;

uint64_t fnv1a(const uint8_t* p, size_t n) {
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
  return h;
}

struct Writer {
  std::vector<uint8_t> buf;
  void raw(const void* p, size_t n) { const uint8_t* b = (const uint8_t*)p; buf.insert(buf.end(), b, b + n); }
  template <typename T> void pod(T v) { raw(&v, sizeof(T)); }
  void str(const std::string& s) { pod<uint64_t>(s.size()); raw(s.data(), s.size()); }
};
struct Reader {
  const uint8_t* p;
  size_t n, at = 0;
  bool ok = true;
  bool raw(void* dst, size_t k) { if (!ok || k > n - at) { ok = false; return false; } memcpy(dst, p + at, k); at += k; return true; }
  template <typename T> T pod() { T v{}; raw(&v, sizeof(T)); return v; }
  std::string str() { uint64_t k = pod<uint64_t>(); if (!ok || k > n - at) { ok = false; return std::string(); } std::string s((const char*)p + at, (size_t)k); at += (size_t)k; return s; }
};

int64_t const_bytes(const _odla_value* v) {
  int64_t e = elem_size(v->type.element_type);
  return e > 0 ? numel(v->type.shape) * e : 0;
}

}  // namespace

extern "C" {

odla_status odla_StoreExecutable(odla_resource_location location, odla_executable executable) {
  if (location.location_type != ODLA_LOCATION_PATH || !location.location || !executable) return ODLA_INVALID_PARAM;  // like odla_tensorrt.cc:539
  _odla_computation* c = (_odla_computation*)executable;
  if (!c->first_error.empty()) return c->error_status;
  Writer w;
  // items
  w.pod<int32_t>(c->float_mode); w.pod<int32_t>(c->n_gpus); w.pod<uint8_t>(c->use_graph ? 1 : 0); w.pod<int32_t>(c->sub_batches);
  // The quantisation table as it was handed over.  Once it has been folded into the graph the nodes below already
  // are in quantise / dequantise form and the table must not be applied a second time.
  w.pod<uint8_t>(c->quant_applied ? 1 : 0);
  w.pod<uint64_t>(c->quant_applied ? 0 : c->quant_table.size());
  if (!c->quant_applied)
    for (auto& q : c->quant_table) { w.str(q.value_id ? (const char*)q.value_id : ""); w.pod<int32_t>(q.ch_idx); w.pod<float>(q.scale); w.pod<float>(q.offset); w.pod<float>(q.min); w.pod<float>(q.max); }
  // nodes
  w.pod<uint64_t>(c->nodes.size());
  for (auto& np : c->nodes) {
    const _odla_value* v = np.get();
    w.str(v->name);
    w.pod<int32_t>((int32_t)v->kind); w.pod<int32_t>((int32_t)v->type.element_type); w.pod<int32_t>(v->type.shape.size);
    for (int i = 0; i < v->type.shape.size; ++i) w.pod<int64_t>(v->type.shape.dims[i]);
    w.pod<uint32_t>((uint32_t)v->in.size());
    for (auto i : v->in) w.pod<int32_t>(i ? i->index : -1);
    w.pod<uint32_t>((uint32_t)v->ia.size());
    for (auto a : v->ia) w.pod<int64_t>(a);
    w.pod<uint32_t>((uint32_t)v->fa.size());
    for (auto a : v->fa) w.pod<float>(a);
    w.pod<uint8_t>(v->is_output ? 1 : 0);
    const int64_t nb = v->kind == OP_CONST && v->host ? const_bytes(v) : 0;
    w.pod<int64_t>(nb);
    if (nb) w.raw(v->host, (size_t)nb);
  }
  w.pod<uint64_t>(c->args.size());
  for (auto a : c->args) w.pod<int32_t>(a->index);
  w.pod<uint64_t>(c->outs.size());
  for (auto o : c->outs) w.pod<int32_t>(o->index);
  // prepared constants (present once the computation has been planned or compiled)
  {
    std::lock_guard<std::mutex> lock(c->prepared_mutex);
    w.pod<uint64_t>(c->prepared.size());
    for (auto& kv : c->prepared) { w.str(kv.first); w.pod<uint64_t>(kv.second->size()); w.raw(kv.second->data(), kv.second->size()); }
  }
  const uint64_t hash = fnv1a(w.buf.data(), w.buf.size());
  std::ofstream f((const char*)location.location, std::ios::binary);
  if (!f) { B2_ERR("odla_StoreExecutable: cannot open '%s'", (const char*)location.location); return ODLA_FAILURE; }
  f.write(kMagic, 8);
  f.write((const char*)&kVersion, 4);
  f.write((const char*)&hash, 8);
  f.write((const char*)w.buf.data(), (std::streamsize)w.buf.size());
  return f.fail() ? ODLA_FAILURE : ODLA_SUCCESS;
}

odla_status odla_LoadExecutable(odla_resource_location location, odla_device, odla_executable* executable) {
  if (!executable) return ODLA_INVALID_PARAM;
  *executable = nullptr;
  std::vector<uint8_t> file;
  const uint8_t* data = nullptr;
  size_t size = 0;
  if (location.location_type == ODLA_LOCATION_PATH && location.location) {
    std::ifstream f((const char*)location.location, std::ios::binary);
    if (!f) { B2_ERR("odla_LoadExecutable: cannot open '%s'", (const char*)location.location); return ODLA_FAILURE; }
    f.seekg(0, std::ios::end);
    file.resize((size_t)f.tellg());
    f.seekg(0, std::ios::beg);
    f.read((char*)file.data(), (std::streamsize)file.size());
    if (!f) return ODLA_FAILURE;
    data = file.data(); size = file.size();
  } else if (location.location_type == ODLA_LOCATION_MEMORY && location.location) {
    data = (const uint8_t*)location.location; size = (size_t)location.size;
  } else return ODLA_FAILURE;
  if (size < 20 || memcmp(data, kMagic, 8) != 0) { B2_ERR("odla_LoadExecutable: not an odla_b200 executable"); return ODLA_FAILURE; }
  uint32_t version; uint64_t hash;
  memcpy(&version, data + 8, 4); memcpy(&hash, data + 12, 8);
  if (version != kVersion) { B2_ERR("odla_LoadExecutable: file version %u, this library reads version %u", version, kVersion); return ODLA_FAILURE; }
  if (fnv1a(data + 20, size - 20) != hash) { B2_ERR("odla_LoadExecutable: the file is damaged (checksum mismatch)"); return ODLA_FAILURE; }
  Reader r{data + 20, size - 20};

  odla_computation c = nullptr;
  if (odla_CreateComputation(&c) != ODLA_SUCCESS) return ODLA_FAILURE;   // becomes the current computation, as in the reference
  auto bail = [&](const char* what) { B2_ERR("odla_LoadExecutable: %s", what); odla_DestroyComputation(c); return ODLA_FAILURE; };
  c->float_mode = r.pod<int32_t>(); c->n_gpus = r.pod<int32_t>(); c->use_graph = r.pod<uint8_t>() != 0; c->sub_batches = r.pod<int32_t>();
  c->quant_applied = r.pod<uint8_t>() != 0;
  const uint64_t nq = r.pod<uint64_t>();
  if (!r.ok || nq > (1u << 24)) return bail("truncated header");
  for (uint64_t i = 0; i < nq; ++i) {
    odla_value_quant_info q{};
    c->quant_names.emplace_back(r.str());
    q.value_id = (odla_value_id)c->quant_names.back().c_str();
    q.ch_idx = r.pod<int32_t>(); q.scale = r.pod<float>(); q.offset = r.pod<float>(); q.min = r.pod<float>(); q.max = r.pod<float>();
    c->quant_table.push_back(q);
  }
  const uint64_t nn = r.pod<uint64_t>();
  if (!r.ok || nn > (1u << 26)) return bail("truncated node list");
  for (uint64_t k = 0; k < nn; ++k) {
    auto v = std::make_unique<_odla_value>();
    v->name = r.str();
    v->kind = (OpKind)r.pod<int32_t>();
    v->type.element_type = (odla_element_type)r.pod<int32_t>();
    v->type.shape.size = r.pod<int32_t>();
    if (!r.ok || v->type.shape.size < 0 || v->type.shape.size > ODLA_MAX_DIMENSION) return bail("bad shape");
    for (int i = 0; i < v->type.shape.size; ++i) v->type.shape.dims[i] = r.pod<int64_t>();
    const uint32_t ni = r.pod<uint32_t>();
    if (!r.ok || ni > 4096) return bail("bad operand count");
    for (uint32_t i = 0; i < ni; ++i) {
      const int32_t idx = r.pod<int32_t>();
      if (idx >= (int32_t)k) return bail("operand refers to a later node");
      v->in.push_back(idx < 0 ? nullptr : c->nodes[(size_t)idx].get());
    }
    const uint32_t nia = r.pod<uint32_t>();
    if (!r.ok || nia > 4096) return bail("bad attribute count");
    for (uint32_t i = 0; i < nia; ++i) v->ia.push_back(r.pod<int64_t>());
    const uint32_t nfa = r.pod<uint32_t>();
    if (!r.ok || nfa > 4096) return bail("bad attribute count");
    for (uint32_t i = 0; i < nfa; ++i) v->fa.push_back(r.pod<float>());
    v->is_output = r.pod<uint8_t>() != 0;
    const int64_t nb = r.pod<int64_t>();
    if (!r.ok || nb < 0 || (size_t)nb > r.n - r.at) return bail("truncated constant");
    if (nb) {
      if (nb != const_bytes(v.get())) return bail("constant size does not match its type");
      auto bytes = std::make_unique<std::vector<uint8_t>>(r.p + r.at, r.p + r.at + nb);
      r.at += (size_t)nb;
      v->host = bytes->data();
      c->owned_consts.push_back(std::move(bytes));
    }
    v->index = (int)k;
    c->by_name[v->name] = v.get();
    c->nodes.push_back(std::move(v));
  }
  const uint64_t na = r.pod<uint64_t>();
  for (uint64_t i = 0; i < na && r.ok; ++i) { const int32_t idx = r.pod<int32_t>(); if (idx < 0 || (uint64_t)idx >= nn) return bail("bad argument index"); c->args.push_back(c->nodes[(size_t)idx].get()); }
  const uint64_t no = r.pod<uint64_t>();
  for (uint64_t i = 0; i < no && r.ok; ++i) { const int32_t idx = r.pod<int32_t>(); if (idx < 0 || (uint64_t)idx >= nn) return bail("bad output index"); c->outs.push_back(c->nodes[(size_t)idx].get()); }
  const uint64_t np = r.pod<uint64_t>();
  for (uint64_t i = 0; i < np && r.ok; ++i) {
    std::string key = r.str();
    const uint64_t nb = r.pod<uint64_t>();
    if (!r.ok || nb > r.n - r.at) return bail("truncated prepared constant");
    c->prepared[key] = std::make_shared<std::vector<uint8_t>>(r.p + r.at, r.p + r.at + nb);
    r.at += (size_t)nb;
  }
  if (!r.ok) return bail("truncated file");
  c->planned = false;
  *executable = (odla_executable)c;
  return ODLA_SUCCESS;
}

/* Extension: how often planning found a constant already prepared / had to prepare it (tests of the executable file). */
void odla_b200_PreparedConstantStats(odla_computation c, long long* hits, long long* misses, long long* entries) {
  if (!c) return;
  std::lock_guard<std::mutex> lock(c->prepared_mutex);
  if (hits) *hits = c->prepared_hits;
  if (misses) *misses = c->prepared_misses;
  if (entries) *entries = (long long)c->prepared.size();
}

}  // extern "C"
