// .lutmac loader: replaces load_lutmac (src/format.cpp:292-505) and the tensor-to-slot mapping
// of load_model (src/model.cpp:576-699).  The file is "LUTMAC01", u32 version (1), u32 header
// size, an ad-hoc JSON header, zero padding to a 256-byte boundary, then the raw block arrays
// (the reference's structs, little endian) at the offsets the header lists.  The parser
// follows the reference's substring search, quirks included: config keys are looked up in the
// whole header, "quant_bits": 1.58 of ternary tensors is read as a float and truncated to 1,
// max_position_embeddings is never read back (the cache keeps the default 2048 positions).
// Block arrays go straight from the file to lmb_weight_upload (re-tiling + one host-to-device
// copy per tensor).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

struct TensorEntry {
  std::string name;
  int kind = -1;  // block kind, -1 = raw fp32
  int quant_bits = 2;
  std::vector<size_t> shape;
  size_t num_blocks = 0, offset = 0;
};

std::string js_string(const std::string &j, const std::string &key) {  // format.cpp:62-77
  size_t k = j.find("\"" + key + "\"");
  if (k == std::string::npos) return "";
  size_t a = j.find("\"", k + key.size() + 2);
  if (a == std::string::npos) return "";
  size_t b = j.find("\"", a + 1);
  if (b == std::string::npos) return "";
  return j.substr(a + 1, b - a - 1);
}

bool js_number(const std::string &j, const std::string &key, std::string *out) {  // format.cpp:80-115
  size_t k = j.find("\"" + key + "\"");
  if (k == std::string::npos) return false;
  size_t colon = j.find(":", k);
  size_t a = j.find_first_not_of(" \t\n\r", colon + 1);
  size_t b = j.find_first_of(",}\n\r", a);
  if (a == std::string::npos) return false;
  *out = j.substr(a, b - a);
  return true;
}

long js_int(const std::string &j, const std::string &key) {
  std::string s;
  if (!js_number(j, key, &s)) return 0;
  char *end = nullptr;
  long v = std::strtol(s.c_str(), &end, 10);
  return end == s.c_str() ? 0 : v;
}

float js_float(const std::string &j, const std::string &key) {
  std::string s;
  if (!js_number(j, key, &s)) return 0.0f;
  char *end = nullptr;
  float v = std::strtof(s.c_str(), &end);
  return end == s.c_str() ? 0.0f : v;
}

bool has(const std::string &s, const char *needle) { return s.find(needle) != std::string::npos; }

}  // namespace

struct lmb_file {
  FILE *fp = nullptr;
  std::string header;
  size_t data_start = 0, file_size = 0;
  std::string model_type;
  size_t vocab = 0, hidden = 0, inter = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0;
  float eps = 1e-5f, theta = 10000.0f, rope_factor = 1.0f;
  int activation = 2;
  std::vector<TensorEntry> tensors;
};

extern "C" {

int lmb_file_close(lmb_file *f) {
  if (!f) return LMB_OK;
  if (f->fp) std::fclose(f->fp);
  delete f;
  return LMB_OK;
}

int lmb_file_open(const char *path, lmb_file **out) {
  using namespace lmb;
  LMB_REQUIRE(path && out, "lmb_file_open: null argument");
  *out = nullptr;
  lmb_file *f = new (std::nothrow) lmb_file();
  if (!f) return LMB_ERR_ALLOC;
  auto fail = [&](const char *msg) {
    set_last_error(std::string("lmb_file_open: ") + msg + " (" + path + ")");
    lmb_file_close(f);
    return LMB_ERR_FORMAT;
  };
  f->fp = std::fopen(path, "rb");
  if (!f->fp) return fail("cannot open file");
  std::fseek(f->fp, 0, SEEK_END);
  f->file_size = size_t(std::ftell(f->fp));
  std::fseek(f->fp, 0, SEEK_SET);
  char magic[8];
  uint32_t version = 0, header_size = 0;
  if (std::fread(magic, 1, 8, f->fp) != 8 || std::memcmp(magic, "LUTMAC01", 8) != 0) return fail("bad magic");  // :299-302
  if (std::fread(&version, 4, 1, f->fp) != 1 || version != 1) return fail("unsupported format version");       // :305-308
  if (std::fread(&header_size, 4, 1, f->fp) != 1 || 16 + size_t(header_size) > f->file_size) return fail("truncated header");
  f->header.assign(header_size, ' ');
  if (std::fread(&f->header[0], 1, header_size, f->fp) != header_size) return fail("truncated header");
  const std::string &h = f->header;
  f->model_type = js_string(h, "model_type");  // :321-342
  f->vocab = size_t(js_int(h, "vocab_size"));
  f->hidden = size_t(js_int(h, "hidden_size"));
  f->inter = size_t(js_int(h, "intermediate_size"));
  f->layers = size_t(js_int(h, "num_hidden_layers"));
  f->heads = size_t(js_int(h, "num_attention_heads"));
  f->kv_heads = size_t(js_int(h, "num_key_value_heads"));
  f->eps = js_float(h, "rms_norm_eps");
  f->theta = js_float(h, "rope_theta");
  f->rope_factor = js_float(h, "rope_scaling_factor");
  if (f->rope_factor <= 0.0f) f->rope_factor = 1.0f;
  f->head_dim = size_t(js_int(h, "head_dim"));
  f->activation = int(js_int(h, "activation"));
  if (f->vocab == 0) return fail("header has no vocab_size");  // :344-345
  size_t pos = h.find("\"tensors\": [");
  if (pos == std::string::npos) return fail("header has no tensor list");
  f->data_start = 16 + header_size + ((256 - ((16 + header_size) % 256)) % 256);  // :354-357
  while (true) {  // :359-502
    size_t ob = h.find("{", pos);
    if (ob == std::string::npos) break;
    size_t cb = h.find("}", ob);
    if (cb == std::string::npos) return fail("unterminated tensor entry");
    const std::string tj = h.substr(ob, cb - ob + 1);
    TensorEntry t;
    t.name = js_string(tj, "name");
    t.num_blocks = size_t(js_int(tj, "num_blocks"));
    if (has(tj, "\"type\": \"int8\"")) t.kind = LMB_INT8;
    else if (has(tj, "\"type\": \"int6\"")) t.kind = LMB_INT6;
    else if (has(tj, "\"type\": \"int5\"")) t.kind = LMB_INT5;
    else if (has(tj, "\"type\": \"int4\"")) t.kind = LMB_INT4;
    else if (has(tj, "\"type\": \"int3\"")) t.kind = LMB_INT3;
    else if (has(tj, "\"type\": \"int2\"")) t.kind = LMB_INT2;
    else if (has(tj, "\"type\": \"binary\"")) t.kind = LMB_BINARY;
    else if (has(tj, "\"type\": \"ternary\"") || has(tj, "\"type\": \"quantized\"") || t.num_blocks > 0) t.kind = LMB_TERNARY;
    std::string qb;
    if (js_number(tj, "quant_bits", &qb)) t.quant_bits = int(std::strtof(qb.c_str(), nullptr));  // 1.58 -> 1 (:394-406)
    size_t ss = tj.find("\"shape\": [");
    if (ss != std::string::npos) {
      size_t se = tj.find("]", ss);
      if (se == std::string::npos) return fail("unterminated shape list");
      std::string body = tj.substr(ss + 10, se - ss - 10);
      size_t p2 = 0;
      while (p2 < body.size()) {
        size_t comma = body.find(",", p2);
        std::string seg = body.substr(p2, comma == std::string::npos ? std::string::npos : comma - p2);
        char *end = nullptr;
        unsigned long v = std::strtoul(seg.c_str(), &end, 10);
        if (end != seg.c_str()) t.shape.push_back(size_t(v));
        if (comma == std::string::npos) break;
        p2 = comma + 1;
      }
    }
    const long rel = js_int(tj, "offset");
    if (rel < 0) return fail("negative tensor offset");
    t.offset = f->data_start + size_t(rel);
    // The header is not trusted: the payload must lie inside the file and a 2-D block tensor must
    // hold exactly shape[0] * ceil(shape[1] / 256) blocks (what the upload will read).
    {
      const size_t lim = size_t(1) << 40;  // keeps the products below free of overflow
      size_t bytes = 0;
      if (t.kind >= 0) {
        if (t.num_blocks > lim) return fail("implausible block count");
        bytes = t.num_blocks * size_t(lmb::kind_info(t.kind).ref_bytes);
        if (t.shape.size() == 2) {
          if (t.shape[0] == 0 || t.shape[1] == 0 || t.shape[0] > lim || t.shape[1] > lim) return fail("bad tensor shape");
          const size_t bpr = (t.shape[1] + 255) / 256;
          if (t.shape[0] > lim / bpr || t.num_blocks != t.shape[0] * bpr) return fail("num_blocks does not match the tensor shape");
        }
      } else {
        bytes = sizeof(float);
        for (size_t sdim : t.shape) {
          if (sdim > lim || (sdim != 0 && bytes > lim / sdim)) return fail("bad tensor shape");
          bytes *= sdim;
        }
      }
      if (t.offset > f->file_size || bytes > f->file_size - t.offset) return fail("tensor data runs past the end of the file");
    }
    f->tensors.push_back(t);
    pos = cb + 1;
  }
  *out = f;
  return LMB_OK;
}

int lmb_file_config(const lmb_file *f, lmb_model_config *cfg) {
  using namespace lmb;
  LMB_REQUIRE(f && cfg, "lmb_file_config: null argument");
  std::memset(cfg, 0, sizeof(*cfg));
  cfg->vocab_size = f->vocab;
  cfg->hidden_size = f->hidden;
  cfg->intermediate_size = f->inter;
  cfg->num_hidden_layers = f->layers;
  cfg->num_attention_heads = f->heads;
  cfg->num_key_value_heads = f->kv_heads;
  cfg->head_dim = f->head_dim > 0 ? f->head_dim : (f->heads ? f->hidden / f->heads : 0);  // types.hpp:585-588
  cfg->max_seq_len = 2048;  // max_position_embeddings is written but never parsed back (types.hpp:558)
  cfg->rope_theta = f->theta;
  cfg->rope_scaling_factor = f->rope_factor;
  cfg->rms_norm_eps = f->eps;
  cfg->max_batch = 1;
  cfg->tp_rank = 0;
  cfg->tp_size = 1;
  cfg->gemma = f->model_type == "gemma" ? 1 : 0;                 // model.cpp:255,294,390,436
  cfg->activation = f->activation == 1 ? LMB_ACT_GELU : LMB_ACT_SILU;  // ActivationType::GELU = 1; everything else takes the SiLU branch (model.cpp:409-417)
  return LMB_OK;
}

int lmb_file_tensor_count(const lmb_file *f, size_t *n) {
  using namespace lmb;
  LMB_REQUIRE(f && n, "lmb_file_tensor_count: null argument");
  *n = f->tensors.size();
  return LMB_OK;
}

int lmb_file_tensor_info(const lmb_file *f, size_t i, const char **name, int *kind, int *quant_bits, size_t *dim0,
                         size_t *dim1, size_t *num_blocks) {
  using namespace lmb;
  LMB_REQUIRE(f && i < f->tensors.size(), "lmb_file_tensor_info: bad argument");
  const TensorEntry &t = f->tensors[i];
  if (name) *name = t.name.c_str();
  if (kind) *kind = t.kind;
  if (quant_bits) *quant_bits = t.quant_bits;
  if (dim0) *dim0 = t.shape.size() > 0 ? t.shape[0] : 0;
  if (dim1) *dim1 = t.shape.size() > 1 ? t.shape[1] : 0;
  if (num_blocks) *num_blocks = t.num_blocks;
  return LMB_OK;
}

int lmb_file_read_tensor(lmb_file *f, size_t i, void *dst, size_t dst_bytes) {
  using namespace lmb;
  LMB_REQUIRE(f && dst && i < f->tensors.size(), "lmb_file_read_tensor: bad argument");
  const TensorEntry &t = f->tensors[i];
  size_t bytes = 0;
  if (t.kind >= 0) bytes = t.num_blocks * size_t(kind_info(t.kind).ref_bytes);
  else {
    bytes = sizeof(float);
    for (size_t s : t.shape) bytes *= s;
  }
  if (bytes > dst_bytes) {
    set_last_error("lmb_file_read_tensor: destination too small");
    return LMB_ERR_ARG;
  }
  if (t.offset + bytes > f->file_size) {
    set_last_error("lmb_file_read_tensor: tensor '" + t.name + "' runs past the end of the file");
    return LMB_ERR_FORMAT;
  }
  std::fseek(f->fp, long(t.offset), SEEK_SET);
  if (std::fread(dst, 1, bytes, f->fp) != bytes) {
    set_last_error("lmb_file_read_tensor: short read");
    return LMB_ERR_FORMAT;
  }
  return LMB_OK;
}

// load_model (src/model.cpp:576-699): names -> slots, norms and biases copied when their length
// fits, lm_head tied to the embedding when the file has none.
int lmb_model_load(lmb_ctx *ctx, const char *path, size_t max_batch, size_t max_seq, int tp_rank, int tp_size,
                   lmb_model **out) {
  using namespace lmb;
  LMB_REQUIRE(ctx && path && out, "lmb_model_load: null argument");
  *out = nullptr;
  lmb_file *f = nullptr;
  int st = lmb_file_open(path, &f);
  if (st != LMB_OK) return st;
  lmb_model_config cfg;
  lmb_file_config(f, &cfg);
  cfg.max_batch = max_batch ? max_batch : 1;
  if (max_seq) cfg.max_seq_len = max_seq;
  cfg.tp_rank = tp_rank;
  cfg.tp_size = tp_size > 0 ? tp_size : 1;
  lmb_model *m = nullptr;
  st = lmb_model_create(ctx, &cfg, &m);
  std::vector<uint8_t> buf;
  bool have_head = false;
  int embed_idx = -1;
  for (size_t i = 0; i < f->tensors.size() && st == LMB_OK; ++i) {
    const TensorEntry &t = f->tensors[i];
    const std::string &n = t.name;
    size_t bytes = sizeof(float);
    if (t.kind >= 0) bytes = t.num_blocks * size_t(kind_info(t.kind).ref_bytes);
    else for (size_t s : t.shape) bytes *= s;
    int slot = -1, vec = -1, layer = 0;
    if (n == "embed_tokens" || n == "token_embeddings.weight" || n == "model.embed_tokens.weight") slot = LMB_SLOT_EMBED;
    else if (n == "norm.weight" || n == "model.norm.weight") vec = LMB_VEC_FINAL_NORM;
    else if (n == "lm_head.weight" || n == "output.weight") slot = LMB_SLOT_LM_HEAD;
    else if (has(n, "layers.")) {
      size_t a = n.find("layers.") + 7, b = n.find(".", a);
      if (b == std::string::npos) continue;
      layer = std::atoi(n.substr(a, b - a).c_str());
      if (layer < 0 || size_t(layer) >= cfg.num_hidden_layers) continue;
      if (has(n, "input_layernorm.weight")) vec = LMB_VEC_INPUT_NORM;
      else if (has(n, "post_attention_layernorm.weight")) vec = LMB_VEC_POST_NORM;
      else if (has(n, "self_attn.q_proj.weight")) slot = LMB_SLOT_Q;
      else if (has(n, "self_attn.k_proj.weight")) slot = LMB_SLOT_K;
      else if (has(n, "self_attn.v_proj.weight")) slot = LMB_SLOT_V;
      else if (has(n, "self_attn.o_proj.weight")) slot = LMB_SLOT_O;
      else if (has(n, "self_attn.q_proj.bias")) vec = LMB_VEC_Q_BIAS;
      else if (has(n, "self_attn.k_proj.bias")) vec = LMB_VEC_K_BIAS;
      else if (has(n, "self_attn.v_proj.bias")) vec = LMB_VEC_V_BIAS;
      else if (has(n, "mlp.gate_proj.weight")) slot = LMB_SLOT_GATE;
      else if (has(n, "mlp.up_proj.weight")) slot = LMB_SLOT_UP;
      else if (has(n, "mlp.down_proj.weight")) slot = LMB_SLOT_DOWN;
    }
    if (slot < 0 && vec < 0) continue;
    buf.resize(bytes);
    st = lmb_file_read_tensor(f, i, buf.data(), buf.size());
    if (st != LMB_OK) break;
    if (vec >= 0) {
      if (t.kind >= 0) continue;  // quantised norms / biases are ignored by the reference too
      const size_t cnt = bytes / sizeof(float);
      const size_t want = vec == LMB_VEC_Q_BIAS ? cfg.num_attention_heads * cfg.head_dim
                        : (vec == LMB_VEC_K_BIAS || vec == LMB_VEC_V_BIAS) ? cfg.num_key_value_heads * cfg.head_dim
                                                                           : cfg.hidden_size;
      if (cnt != want) continue;  // size mismatch: the reference keeps its default
      st = lmb_model_set_vector(m, layer, vec, reinterpret_cast<const float *>(buf.data()), cnt);
    } else {
      if (t.kind < 0 || t.shape.size() != 2) {
        set_last_error("lmb_model_load: tensor '" + n + "' is not a 2-D quantised tensor");
        st = LMB_ERR_FORMAT;
        break;
      }
      st = lmb_model_set_weight(m, layer, slot, t.kind, t.quant_bits, buf.data(), t.shape[0], t.shape[1]);
      if (slot == LMB_SLOT_LM_HEAD) have_head = true;
      if (slot == LMB_SLOT_EMBED) embed_idx = int(i);
    }
  }
  if (st == LMB_OK && !have_head && embed_idx >= 0 && cfg.tp_size == 1) {  // tied head (model.cpp:667-689)
    st = model_tie_head(m);
  } else if (st == LMB_OK && !have_head && embed_idx >= 0) {  // sharded: every rank keeps its rows of the head
    const TensorEntry &t = f->tensors[size_t(embed_idx)];
    buf.resize(t.num_blocks * size_t(kind_info(t.kind).ref_bytes));
    st = lmb_file_read_tensor(f, size_t(embed_idx), buf.data(), buf.size());
    if (st == LMB_OK) st = lmb_model_set_weight(m, 0, LMB_SLOT_LM_HEAD, t.kind, t.quant_bits, buf.data(), t.shape[0], t.shape[1]);
  }
  lmb_file_close(f);
  if (st != LMB_OK) {
    lmb_model_destroy(m);
    return st;
  }
  *out = m;
  return LMB_OK;
}

}  // extern "C"
