// Native GGUF loader: memory-map the file, read the header, the metadata and the tensor directory, and stream the
// tensors of a Llama-architecture model to the device in their stored type (raw float16 stays float16: no widening
// pass on the CPU). It drives the same public entry points a managed host would (nfai_model_create / tensor_* /
// finalize), so it adds no second upload path.
//
// What it stands in for: NFAI.GGUF/Parser.cs (header and magic :130-143, the 13 metadata value types incl. nested
// arrays :145-236, tensor directory :244-307, data alignment :32-33,125-128) plus the per-element half->float loop
// and managed 10 MiB arrays of NFAI.Core/AbstractComputeCollection.cs:36-79 and the whole-tensor staging of
// NFAI.Vulkan/VulkanBufferManager.cs:105-194.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/nfai_cuda.h"

struct nfai_ctx;
namespace nfai {
int ctx_fail(nfai_ctx* c, int code, const char* message);
}

namespace {

struct Reader {
  const unsigned char* p;
  size_t n, off = 0;
  bool bad = false;
  template <typename T>
  T get() {
    T v{};
    if (sizeof(T) > n - off) { bad = true; return v; }  // off <= n always holds
    memcpy(&v, p + off, sizeof(T));
    off += sizeof(T);
    return v;
  }
  std::string str() {
    uint64_t len = get<uint64_t>();
    if (bad || len > n - off) { bad = true; return std::string(); }
    std::string s((const char*)p + off, (size_t)len);
    off += len;
    return s;
  }
};

struct MetaValue {
  int type = -1;
  double num = 0;  // every scalar as a double (exact for the integer ranges that matter here)
  std::string str;
};

size_t scalar_size(uint32_t t) {
  switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
  }
}

bool read_value(Reader& r, uint32_t type, MetaValue* out, int depth) {
  if (depth > 4) return false;
  switch (type) {
    case 0: { auto v = r.get<uint8_t>(); if (out) out->num = v; break; }
    case 1: { auto v = r.get<int8_t>(); if (out) out->num = v; break; }
    case 2: { auto v = r.get<uint16_t>(); if (out) out->num = v; break; }
    case 3: { auto v = r.get<int16_t>(); if (out) out->num = v; break; }
    case 4: { auto v = r.get<uint32_t>(); if (out) out->num = v; break; }
    case 5: { auto v = r.get<int32_t>(); if (out) out->num = v; break; }
    case 6: { auto v = r.get<float>(); if (out) out->num = v; break; }
    case 7: { auto v = r.get<uint8_t>(); if (out) out->num = v != 0; break; }
    case 8: { std::string s = r.str(); if (out) out->str = s; break; }
    case 9: {
      uint32_t et = r.get<uint32_t>();
      uint64_t cnt = r.get<uint64_t>();
      if (r.bad) return false;
      size_t es = scalar_size(et);
      if (es) {  // skip arrays of scalars in one step
        if (cnt > (r.n - r.off) / es) return false;  // no product that could wrap
        r.off += es * cnt;
      } else {
        for (uint64_t i = 0; i < cnt; ++i)
          if (!read_value(r, et, nullptr, depth + 1)) return false;
      }
      break;
    }
    case 10: { auto v = r.get<uint64_t>(); if (out) out->num = (double)v; break; }
    case 11: { auto v = r.get<int64_t>(); if (out) out->num = (double)v; break; }
    case 12: { auto v = r.get<double>(); if (out) out->num = v; break; }
    default: return false;
  }
  if (out) out->type = (int)type;
  return !r.bad;
}

struct TensorInfo {
  std::vector<uint64_t> shape;
  uint32_t ggml_type = 0;
  uint64_t offset = 0;
};

// Everything that can be decided from the file alone, before a device is touched.
struct ParsedFile {
  nfai_hparams hp;
  std::map<std::string, TensorInfo> tensors;
  uint64_t data_start = 0;
  std::vector<std::string> names;  // tensors the model needs, in upload order
};

// Header, metadata, tensor directory and the bounds of every tensor the model needs. Sizes and offsets come from
// the file and are hostile until checked: every comparison is written so that it cannot wrap.
int parse_gguf(const unsigned char* map, size_t fsize, uint32_t kv_cache_size, int kv_dtype, ParsedFile* pf,
               std::string* err) {
  auto bad = [&](const std::string& m) { *err = m; return NFAI_ERR_ARG; };
  Reader r{map, fsize};
  if (r.get<uint32_t>() != 0x46554747u) return bad("not a GGUF file (bad magic)");
  const uint32_t version = r.get<uint32_t>();
  if (version < 2) return bad("GGUF version 1 is not supported");
  const uint64_t n_tensors = r.get<uint64_t>();
  const uint64_t n_kv = r.get<uint64_t>();
  if (r.bad) return bad("truncated GGUF header");
  // every entry takes at least 12 bytes: a count beyond that is a lie, not a reason to loop
  if (n_kv > fsize / 12 || n_tensors > fsize / 12) return bad("GGUF header counts exceed the file size");
  std::map<std::string, MetaValue> meta;
  for (uint64_t i = 0; i < n_kv && !r.bad; ++i) {
    std::string key = r.str();
    uint32_t type = r.get<uint32_t>();
    MetaValue v;
    if (!read_value(r, type, &v, 0)) return bad("malformed GGUF metadata");
    if (type != 9) meta[key] = v;
  }
  for (uint64_t i = 0; i < n_tensors && !r.bad; ++i) {
    std::string name = r.str();
    uint32_t nd = r.get<uint32_t>();
    if (r.bad) break;
    if (nd > 4) return bad("tensor with more than 4 dimensions");
    TensorInfo t;
    for (uint32_t k = 0; k < nd; ++k) t.shape.push_back(r.get<uint64_t>());
    t.ggml_type = r.get<uint32_t>();
    t.offset = r.get<uint64_t>();
    pf->tensors[name] = t;
  }
  if (r.bad) return bad("truncated GGUF directory");
  auto num = [&](const char* key, double dflt) {
    auto it = meta.find(key);
    return it == meta.end() ? dflt : it->second.num;
  };
  {
    auto it = meta.find("general.architecture");
    if (it == meta.end() || it->second.str != "llama")  // LlamaModelFactory.cs:36-43
      return bad("general.architecture is not \"llama\"");
  }
  const double align_d = num("general.alignment", 32);
  if (!(align_d >= 1 && align_d <= 1048576)) return bad("general.alignment must be a power of two between 1 and 2^20");
  const uint64_t alignment = (uint64_t)align_d;
  if ((alignment & (alignment - 1)) != 0) return bad("general.alignment must be a power of two between 1 and 2^20");
  if (r.off > fsize - (alignment - 1 < fsize ? alignment - 1 : fsize)) {
    // rounding up would pass the end of the file: there is no data section
    return bad("GGUF file has no tensor data");
  }
  pf->data_start = (r.off + alignment - 1) / alignment * alignment;

  auto find = [&](const std::string& name) -> const TensorInfo* {
    auto it = pf->tensors.find(name);
    return it == pf->tensors.end() ? nullptr : &it->second;
  };
  const TensorInfo* embd = find("token_embd.weight");
  const TensorInfo* gate0 = find("blk.0.ffn_gate.weight");
  if (!embd || embd->shape.size() != 2 || !gate0 || gate0->shape.size() != 2)
    return bad("token_embd.weight / blk.0.ffn_gate.weight missing");
  auto u32 = [&](double v, uint32_t* out) {  // metadata numbers are doubles: refuse what a uint32 cannot hold
    if (!(v >= 0 && v <= 4294967295.0)) return false;
    *out = (uint32_t)v;
    return true;
  };
  nfai_hparams& hp = pf->hp;
  memset(&hp, 0, sizeof hp);
  if (embd->shape[0] > 0xffffffffull || embd->shape[1] > 0xffffffffull || gate0->shape[1] > 0xffffffffull)
    return bad("tensor dimensions do not fit 32 bits");
  hp.H = (uint32_t)embd->shape[0];
  hp.V = (uint32_t)embd->shape[1];
  hp.F = (uint32_t)gate0->shape[1];
  bool ok = u32(num("llama.block_count", 0), &hp.L) && u32(num("llama.attention.head_count", 0), &hp.qH);
  ok = ok && u32(num("llama.attention.head_count_kv", hp.qH), &hp.kvH);
  ok = ok && u32(num("llama.attention.key_length", hp.qH ? hp.H / hp.qH : 0), &hp.d);
  ok = ok && u32(num("llama.rope.dimension_count", hp.d), &hp.ropeDim);
  if (!ok || hp.L > 4096) return bad("llama.* metadata out of range");
  hp.ctx = kv_cache_size;
  hp.eps = 0.f;
  for (auto& kv : meta)  // the first key that contains "epsilon" (LlamaModel.cs:28)
    if (kv.first.find("epsilon") != std::string::npos) { hp.eps = (float)kv.second.num; break; }
  hp.rope_theta = (float)num("llama.rope.freq_base", 500000.0);
  hp.weight_dtype = embd->ggml_type == 1 ? NFAI_F16 : NFAI_F32;
  hp.kv_dtype = (kv_dtype == NFAI_F16 || kv_dtype == NFAI_F32) ? kv_dtype : hp.weight_dtype;
  hp.tied = find("output.weight") ? 0 : 1;

  pf->names = {"token_embd.weight", "output_norm.weight"};
  if (!hp.tied) pf->names.push_back("output.weight");
  const char* per_layer[] = {"attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down"};
  for (uint32_t l = 0; l < hp.L; ++l)
    for (const char* s : per_layer) pf->names.push_back("blk." + std::to_string(l) + "." + s + ".weight");
  for (const std::string& name : pf->names) {
    const TensorInfo* t = find(name);
    if (!t) return bad("tensor missing in the file: " + name);
    if (t->ggml_type > 1) return bad("tensor is neither F32 nor F16: " + name);
    const uint64_t esz = t->ggml_type == 1 ? 2 : 4;
    uint64_t count = 1;
    for (uint64_t s : t->shape) {
      if (s != 0 && count > (uint64_t)fsize / s) return bad("tensor data beyond the end of the file: " + name);
      count *= s;
    }
    if (count > (uint64_t)fsize / esz) return bad("tensor data beyond the end of the file: " + name);
    const uint64_t bytes = count * esz;
    if (pf->data_start > fsize || t->offset > fsize - pf->data_start || bytes > fsize - pf->data_start - t->offset)
      return bad("tensor data beyond the end of the file: " + name);
  }
  return NFAI_OK;
}

struct Mapping {
  void* map = MAP_FAILED;
  size_t size = 0;
  ~Mapping() { if (map != MAP_FAILED) munmap(map, size); }
};

int map_file(const char* path, Mapping* m, std::string* err) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) { *err = std::string("cannot open ") + path; return NFAI_ERR_ARG; }
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size < 24) {
    close(fd);
    *err = "not a GGUF file (too short)";
    return NFAI_ERR_ARG;
  }
  m->size = (size_t)sb.st_size;
  m->map = mmap(nullptr, m->size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (m->map == MAP_FAILED) { *err = "mmap failed"; return NFAI_ERR_ARG; }
  madvise(m->map, m->size, MADV_SEQUENTIAL);
  return NFAI_OK;
}

}  // namespace

extern "C" int nfai_gguf_probe(const char* path, uint32_t kv_cache_size, nfai_hparams* out, char* err_out, size_t err_bytes) {
  std::string err;
  int rc = NFAI_ERR_ARG;
  try {
    if (!path || !out) {
      err = "bad argument";
    } else {
      Mapping m;
      rc = map_file(path, &m, &err);
      if (rc == NFAI_OK) {
        ParsedFile pf;
        rc = parse_gguf((const unsigned char*)m.map, m.size, kv_cache_size ? kv_cache_size : 1, 0, &pf, &err);
        if (rc == NFAI_OK) *out = pf.hp;
      }
    }
  } catch (const std::bad_alloc&) {
    rc = NFAI_ERR_OOM;
    err = "out of host memory while reading the GGUF directory";
  } catch (const std::exception& e) {
    rc = NFAI_ERR_ARG;
    err = std::string("malformed GGUF file: ") + e.what();
  }
  if (err_out && err_bytes) {
    strncpy(err_out, err.c_str(), err_bytes - 1);
    err_out[err_bytes - 1] = 0;
  }
  return rc;
}

extern "C" int nfai_model_load_gguf(nfai_ctx* ctx, const char* path, uint32_t kv_cache_size, int kv_dtype, nfai_model** out) {
  using nfai::ctx_fail;
  if (!ctx) return NFAI_ERR_ARG;
  if (!path || !out || !kv_cache_size) return ctx_fail(ctx, NFAI_ERR_ARG, "bad argument");
  *out = nullptr;
  nfai_model* model = nullptr;
  // No C++ exception may cross the C boundary: a hostile directory can make a container throw.
  try {
    std::string err;
    Mapping m;
    int rc = map_file(path, &m, &err);
    if (rc != NFAI_OK) return ctx_fail(ctx, rc, err.c_str());
    ParsedFile pf;
    rc = parse_gguf((const unsigned char*)m.map, m.size, kv_cache_size, kv_dtype, &pf, &err);
    if (rc != NFAI_OK) return ctx_fail(ctx, rc, err.c_str());
    rc = nfai_model_create(ctx, &pf.hp, &model);
    if (rc != NFAI_OK) return rc;
    for (const std::string& name : pf.names) {
      const TensorInfo& t = pf.tensors.at(name);
      uint64_t count = 1;
      for (uint64_t s : t.shape) count *= s;  // bounded by the file size (checked by parse_gguf)
      const uint64_t bytes = count * (t.ggml_type == 1 ? 2 : 4);
      const uint64_t begin = pf.data_start + t.offset;
      rc = nfai_model_tensor_begin(model, name.c_str(), t.ggml_type == 1 ? NFAI_F16 : NFAI_F32, t.shape.data(), (int)t.shape.size());
      if (rc == NFAI_OK)
        rc = nfai_model_tensor_chunk(model, (const unsigned char*)m.map + begin, (size_t)bytes);  // staged 16 MiB at a time inside
      if (rc == NFAI_OK) rc = nfai_model_tensor_end(model);
      if (rc != NFAI_OK) break;
    }
    if (rc == NFAI_OK) rc = nfai_model_finalize(model);
    if (rc != NFAI_OK) {
      nfai_model_destroy(model);  // keeps the context's error text
      return rc;
    }
    *out = model;
    return NFAI_OK;
  } catch (const std::bad_alloc&) {
    if (model) nfai_model_destroy(model);
    return ctx_fail(ctx, NFAI_ERR_OOM, "out of host memory while reading the GGUF file");
  } catch (const std::exception& e) {
    if (model) nfai_model_destroy(model);
    return ctx_fail(ctx, NFAI_ERR_ARG, (std::string("malformed GGUF file: ") + e.what()).c_str());
  }
}
