// Readers for the reference's binary snapshots: weights ("RBWTS001", TransformerLm::save_bin /
// load_bin, reference transformer.rs:1809-1932) and Adam moments ("RBOPT001",
// save_optimizer_state / load_optimizer_state, transformer.rs:1675-1753).  Host code: the files are
// walked with fseek, only the tensors of the requested MoE block are read, and they reach the
// device through the same entry points a caller would use (moe_set_weight_f32, moe_set_weight_q8,
// moe_set_moments_f32).  The format is documented in include/moe_b200.h.

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/moe_b200.h"
#include "layer.cuh"

namespace {

// ---------------------------------------------------------------------------
// A small JSON reader: enough for the header serde_json writes (objects, arrays, numbers,
// strings, booleans, null).  Values keep their source text for numbers.
// ---------------------------------------------------------------------------
struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Json> items;
  std::vector<std::pair<std::string, Json>> fields;
  const Json* get(const char* key) const {
    for (const auto& f : fields)
      if (f.first == key) return &f.second;
    return nullptr;
  }
};

struct JsonParser {
  const char* p;
  const char* end;
  bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool lit(const char* s) {
    const size_t n = strlen(s);
    if ((size_t)(end - p) >= n && memcmp(p, s, n) == 0) { p += n; return true; }
    return false;
  }
  std::string string() {
    std::string out;
    if (p >= end || *p != '"') { ok = false; return out; }
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
          case 'u': out += '?'; p += (end - p > 4) ? 4 : 0; break;   // names in this header are ASCII
          default: out += *p;
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= end) { ok = false; return out; }
    ++p;
    return out;
  }
  Json value(int depth = 0) {
    Json v;
    ws();
    if (p >= end || depth > 64) { ok = false; return v; }
    if (*p == '{') {
      v.kind = Json::Object;
      ++p; ws();
      if (p < end && *p == '}') { ++p; return v; }
      while (ok) {
        ws();
        std::string key = string();
        ws();
        if (!ok || p >= end || *p != ':') { ok = false; break; }
        ++p;
        v.fields.emplace_back(std::move(key), value(depth + 1));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; break; }
        ok = false;
      }
    } else if (*p == '[') {
      v.kind = Json::Array;
      ++p; ws();
      if (p < end && *p == ']') { ++p; return v; }
      while (ok) {
        v.items.push_back(value(depth + 1));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; break; }
        ok = false;
      }
    } else if (*p == '"') {
      v.kind = Json::String;
      v.str = string();
    } else if (lit("true")) {
      v.kind = Json::Bool; v.b = true;
    } else if (lit("false")) {
      v.kind = Json::Bool; v.b = false;
    } else if (lit("null")) {
      v.kind = Json::Null;
    } else {
      char* stop = nullptr;
      std::string text(p, (size_t)std::min<ptrdiff_t>(end - p, 64));
      v.num = strtod(text.c_str(), &stop);
      if (stop == text.c_str()) { ok = false; return v; }
      v.kind = Json::Number;
      p += stop - text.c_str();
    }
    return v;
  }
};

void say(char* msg, int len, const char* fmt, ...) {
  if (!msg || len <= 0) return;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, (size_t)len, fmt, ap);
  va_end(ap);
}

struct File {
  FILE* f = nullptr;
  explicit File(const char* path) { f = path ? fopen(path, "rb") : nullptr; }
  ~File() { if (f) fclose(f); }
  bool read(void* dst, size_t n) { return f && fread(dst, 1, n, f) == n; }
  bool u64(uint64_t* v) {
    unsigned char b[8];
    if (!read(b, 8)) return false;
    uint64_t x = 0;
    for (int i = 7; i >= 0; --i) x = (x << 8) | b[i];
    *v = x;
    return true;
  }
  bool skip(uint64_t n) { return f && fseeko(f, (off_t)n, SEEK_CUR) == 0; }
};

bool integer_field(const Json& cfg, const char* key, int64_t* out, char* msg, int len) {
  const Json* v = cfg.get(key);
  if (!v || v->kind != Json::Number || v->num < 0 || v->num != std::floor(v->num)) {
    say(msg, len, "InvalidSnapshot: header field config.%s is missing or not a non-negative integer", key);
    return false;
  }
  *out = (int64_t)v->num;
  return true;
}

// Where the parameters of one block start and how many each block has.
struct Layout {
  std::vector<int64_t> ffn_first;   // index of the first feed-forward parameter of every block
  int64_t total = 0;
};

Layout layout_of(const moe_snapshot_info_t& s) {
  Layout l;
  const int64_t per_linear = s.lora_rank > 0 ? 3 : 1;   // weight (+ down, up)
  int64_t idx = 1;   // embedding
  for (int64_t b = 0; b < s.n_layers; ++b) {
    bool moe = false;
    for (int i = 0; i < s.n_moe_layers; ++i) moe = moe || s.moe_layers[i] == b;
    idx += 1 + 4 * per_linear + 1;   // attention norm, query, key, value, output, feed-forward norm
    l.ffn_first.push_back(idx);
    // the router carries no adapter (moe.rs:502-504)
    idx += moe ? 1 + (3 * s.num_experts + (s.shared_expert ? 3 : 0)) * per_linear : s.dense_ffn_params * per_linear;
  }
  idx += 1;   // final norm
  if (!s.tie_embeddings) idx += 1;   // the LM head is not adapted either
  l.total = idx;
  return l;
}

// Reads magic + header of a weight file and leaves the file positioned at the first parameter.
int open_weights(File& in, moe_snapshot_info_t* s, char* msg, int len) {
  memset(s, 0, sizeof(*s));
  char magic[8];
  if (!in.f) { say(msg, len, "InvalidSnapshot: cannot open the weight file"); return MOE_INVALID_INPUT; }
  if (!in.read(magic, 8) || memcmp(magic, "RBWTS001", 8) != 0) {
    say(msg, len, "InvalidSnapshot: not a RustingBrain weight file");   // transformer.rs:1868-1872
    return MOE_INVALID_INPUT;
  }
  uint64_t hlen = 0;
  if (!in.u64(&hlen) || hlen == 0 || hlen > (64u << 20)) { say(msg, len, "InvalidSnapshot: bad header length"); return MOE_INVALID_INPUT; }
  std::string text(hlen, '\0');
  if (!in.read(&text[0], hlen)) { say(msg, len, "InvalidSnapshot: truncated header"); return MOE_INVALID_INPUT; }
  JsonParser jp{text.data(), text.data() + text.size()};
  const Json root = jp.value();
  const Json* cfg = jp.ok ? root.get("config") : nullptr;
  const Json* prec = jp.ok ? root.get("precision") : nullptr;
  if (!cfg || cfg->kind != Json::Object || !prec || prec->kind != Json::String) {
    say(msg, len, "InvalidSnapshot: the header is not the JSON object save_bin writes");
    return MOE_INVALID_INPUT;
  }
  if (prec->str == "F32") s->precision = MOE_PRECISION_F32;
  else if (prec->str == "Q8") s->precision = MOE_PRECISION_Q8;
  else { say(msg, len, "InvalidSnapshot: unknown precision '%s'", prec->str.c_str()); return MOE_INVALID_INPUT; }
  if (!integer_field(*cfg, "vocab_size", &s->vocab_size, msg, len) || !integer_field(*cfg, "d_model", &s->d_model, msg, len) ||
      !integer_field(*cfg, "n_layers", &s->n_layers, msg, len) || !integer_field(*cfg, "n_heads", &s->n_heads, msg, len) ||
      !integer_field(*cfg, "n_kv_heads", &s->n_kv_heads, msg, len) || !integer_field(*cfg, "head_dim", &s->head_dim, msg, len) ||
      !integer_field(*cfg, "d_ff", &s->d_ff, msg, len) || !integer_field(*cfg, "moe_d_ff", &s->moe_d_ff, msg, len) ||
      !integer_field(*cfg, "num_experts", &s->num_experts, msg, len) ||
      !integer_field(*cfg, "experts_per_token", &s->experts_per_token, msg, len) ||
      !integer_field(*cfg, "max_seq_len", &s->max_seq_len, msg, len))
    return MOE_INVALID_INPUT;
  auto flag = [&](const char* key, int32_t dflt) {
    const Json* v = cfg->get(key);
    return v && v->kind == Json::Bool ? (v->b ? 1 : 0) : dflt;
  };
  auto real = [&](const char* key) {
    const Json* v = cfg->get(key);
    return v && v->kind == Json::Number ? (float)v->num : 0.f;
  };
  s->shared_expert = flag("shared_expert", 0);
  s->tie_embeddings = flag("tie_embeddings", 0);
  s->causal = flag("causal", 1);   // absent in older files: a decoder (transformer.rs:49-52)
  s->aux_loss_weight = real("aux_loss_weight");
  s->router_z_loss_weight = real("router_z_loss_weight");
  s->rope_base = real("rope_base");
  s->rmsnorm_eps = real("rmsnorm_eps");
  const Json* lora = cfg->get("lora");
  if (lora && lora->kind == Json::Object) {
    // the file of an adapted model holds, after every adapted projection, its `down` and `up`
    // (Linear::params_mut, param.rs:859-865)
    const Json* jr = lora->get("rank");
    const Json* ja = lora->get("alpha");
    if (!jr || jr->kind != Json::Number || jr->num < 1 || !ja || ja->kind != Json::Number) {
      say(msg, len, "InvalidSnapshot: config.lora is not a LoraConfig");
      return MOE_INVALID_INPUT;
    }
    s->lora_rank = (int32_t)jr->num;
    s->lora_alpha = (float)ja->num;
  }
  const Json* ml = cfg->get("moe_layers");
  if (!ml || ml->kind != Json::Array || ml->items.size() > 256) {
    say(msg, len, "InvalidSnapshot: config.moe_layers is missing or has more than 256 entries");
    return MOE_INVALID_INPUT;
  }
  for (const Json& v : ml->items) {
    if (v.kind != Json::Number || v.num < 0 || v.num >= (double)s->n_layers) {
      say(msg, len, "InvalidSnapshot: config.moe_layers names a block the model does not have");
      return MOE_INVALID_INPUT;
    }
    s->moe_layers[s->n_moe_layers++] = (int32_t)v.num;
  }
  const Json* step = root.get("optimizer_step");
  s->optimizer_step = step && step->kind == Json::Number ? (int64_t)step->num : 0;
  uint64_t count = 0;
  if (!in.u64(&count)) { say(msg, len, "InvalidSnapshot: truncated file (no parameter count)"); return MOE_INVALID_INPUT; }
  s->parameter_count = (int64_t)count;
  // The configuration does not say which dense feed-forward the model uses; the count does.
  const int64_t dense_blocks = s->n_layers - s->n_moe_layers;
  s->dense_ffn_params = 0;
  bool matched = dense_blocks == 0 && layout_of(*s).total == s->parameter_count;
  for (int per = 3; !matched && per >= 2 && dense_blocks > 0; --per) {
    s->dense_ffn_params = per;
    matched = layout_of(*s).total == s->parameter_count;
  }
  if (!matched) {
    say(msg, len, "InvalidSnapshot: weight file holds %lld parameters, this configuration builds a different number",
        (long long)s->parameter_count);   // transformer.rs:1892-1897
    return MOE_INVALID_INPUT;
  }
  return MOE_OK;
}

}  // namespace

namespace {

struct Tensor {
  uint64_t rows = 0, cols = 0;
  std::vector<float> f32;       // F32 files
  std::vector<int8_t> q;        // Q8 files: rows x cols
  std::vector<float> scale;     // Q8 files: one per row
};

uint64_t payload_bytes(int precision, uint64_t rows, uint64_t cols) {
  return precision == MOE_PRECISION_Q8 ? rows * (4 + cols) : rows * cols * 4;
}

bool skip_params(File& in, int precision, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint64_t rows, cols;
    if (!in.u64(&rows) || !in.u64(&cols) || !in.skip(payload_bytes(precision, rows, cols))) return false;
  }
  return true;
}

// Reads one parameter; the shape must be the one the model has (transformer.rs:1904-1909).
int read_param(File& in, int precision, uint64_t want_rows, uint64_t want_cols, Tensor* t, std::string* err) {
  if (!in.u64(&t->rows) || !in.u64(&t->cols)) { *err = "InvalidSnapshot: truncated weight file"; return MOE_INVALID_INPUT; }
  if (t->rows != want_rows || t->cols != want_cols) {
    *err = "InvalidSnapshot: weight file has a " + std::to_string(t->rows) + "x" + std::to_string(t->cols) +
           " parameter where the layer has " + std::to_string(want_rows) + "x" + std::to_string(want_cols);
    return MOE_INVALID_INPUT;
  }
  const size_t n = (size_t)(t->rows * t->cols);
  bool ok = true;
  if (precision == MOE_PRECISION_Q8) {
    t->q.resize(n);
    t->scale.resize((size_t)t->rows);
    for (uint64_t r = 0; r < t->rows && ok; ++r)
      ok = in.read(&t->scale[(size_t)r], 4) && in.read(t->q.data() + (size_t)(r * t->cols), (size_t)t->cols);
  } else {
    t->f32.resize(n);
    ok = in.read(t->f32.data(), n * 4);
  }
  if (!ok) { *err = "InvalidSnapshot: truncated weight file"; return MOE_INVALID_INPUT; }
  return MOE_OK;
}

// Hands one tensor to the layer in whatever form the handle keeps it.
int put_weight(moe_layer_t* L, int which, int expert, int file_precision, Tensor& t) {
  const bool want_q8 = L->precision == MOE_PRECISION_Q8 && which != MOE_W_ROUTER;
  const size_t n = (size_t)(t.rows * t.cols);
  if (want_q8) {
    if (file_precision != MOE_PRECISION_Q8) {
      // the reference's grid: scale = max|row| / 127, round half away from zero, clamp (transformer.rs:514-519)
      t.q.resize(n);
      t.scale.resize((size_t)t.rows);
      for (uint64_t r = 0; r < t.rows; ++r) {
        const float* row = t.f32.data() + (size_t)(r * t.cols);
        float absmax = 0.f;
        for (uint64_t c = 0; c < t.cols; ++c) absmax = std::fmax(absmax, std::fabs(row[c]));
        const float scale = absmax / 127.0f;
        t.scale[(size_t)r] = scale;
        for (uint64_t c = 0; c < t.cols; ++c) {
          float v = scale == 0.f ? 0.f : roundf(row[c] / scale);
          v = v < -127.f ? -127.f : (v > 127.f ? 127.f : v);
          t.q[(size_t)(r * t.cols + c)] = (int8_t)v;
        }
      }
    }
    return moe_set_weight_q8(L, which, expert, t.q.data(), t.scale.data(), (int32_t)t.rows, (int32_t)t.cols);
  }
  if (file_precision == MOE_PRECISION_Q8) {
    t.f32.resize(n);   // load_bin: value = byte as i8 as f32 * scale (transformer.rs:1917-1927)
    for (uint64_t r = 0; r < t.rows; ++r)
      for (uint64_t c = 0; c < t.cols; ++c)
        t.f32[(size_t)(r * t.cols + c)] = (float)t.q[(size_t)(r * t.cols + c)] * t.scale[(size_t)r];
  }
  return moe_set_weight_f32(L, which, expert, t.f32.data(), (int32_t)t.rows, (int32_t)t.cols);
}

int check_block(moe_layer_t* L, const moe_snapshot_info_t& s, int block) {
  bool is_moe = false;
  for (int i = 0; i < s.n_moe_layers; ++i) is_moe = is_moe || s.moe_layers[i] == block;
  if (block < 0 || block >= s.n_layers || !is_moe) {
    L->err = "InvalidInput: block " + std::to_string(block) + " of the file is not a MoE block";
    return MOE_INVALID_INPUT;
  }
  if (s.d_model != L->d || s.num_experts != L->E || s.moe_d_ff != L->F || (s.shared_expert != 0) != L->shared) {
    L->err = "InvalidConfig: the file's MoE blocks are d_model " + std::to_string(s.d_model) + ", " +
             std::to_string(s.num_experts) + " experts, d_ff " + std::to_string(s.moe_d_ff) +
             (s.shared_expert ? " + shared" : "") + "; the handle is " + std::to_string(L->d) + ", " +
             std::to_string(L->E) + ", " + std::to_string(L->F) + (L->shared ? " + shared" : "");
    return MOE_INVALID_CONFIG;
  }
  return MOE_OK;
}

// (which, expert, rows, cols) of the parameters of a MoE feed-forward, in file order (moe.rs:516-525).
struct Entry { int which, expert; uint64_t rows, cols; bool mine; };
std::vector<Entry> moe_entries(const moe_layer_t* L) {
  std::vector<Entry> v;
  const uint64_t d = (uint64_t)L->d, F = (uint64_t)L->F;
  v.push_back({MOE_W_ROUTER, 0, (uint64_t)L->E, d, true});
  for (int e = 0; e < L->E; ++e) {
    const bool mine = e >= L->e0 && e < L->e0 + L->E_local;
    v.push_back({MOE_W_GATE, e, F, d, mine});
    v.push_back({MOE_W_UP, e, F, d, mine});
    v.push_back({MOE_W_DOWN, e, d, F, mine});
  }
  if (L->shared) {
    v.push_back({MOE_W_SHARED_GATE, 0, F, d, true});
    v.push_back({MOE_W_SHARED_UP, 0, F, d, true});
    v.push_back({MOE_W_SHARED_DOWN, 0, d, F, true});
  }
  return v;
}

}  // namespace

extern "C" {

int32_t moe_snapshot_info(const char* weights_path, moe_snapshot_info_t* out, char* message, int32_t message_len) {
  if (!weights_path || !out) { say(message, message_len, "InvalidInput: null argument"); return MOE_INVALID_INPUT; }
  File in(weights_path);
  return open_weights(in, out, message, message_len);
}

int32_t moe_load_snapshot_layer(moe_layer_t* L, const char* weights_path, int32_t block_index) {
  if (!L) return MOE_INVALID_INPUT;
  if (L->status != MOE_OK) return MOE_POISONED;
  if (!weights_path) { L->err = "InvalidInput: null path"; return MOE_INVALID_INPUT; }
  File in(weights_path);
  moe_snapshot_info_t s;
  char msg[256] = {0};
  int rc = open_weights(in, &s, msg, sizeof(msg));
  if (rc != MOE_OK) { L->err = msg; return rc; }
  if ((rc = check_block(L, s, block_index)) != MOE_OK) return rc;
  const Layout lay = layout_of(s);
  if (!skip_params(in, s.precision, lay.ffn_first[(size_t)block_index])) {
    L->err = "InvalidSnapshot: truncated weight file";
    return MOE_INVALID_INPUT;
  }
  // adapters in the file go into the layer's adapters when it has some of the same rank and alpha;
  // a layer without adapters takes the base weights only
  const bool file_lora = s.lora_rank > 0;
  const bool take_lora = file_lora && L->lora_rank == s.lora_rank && L->lora_alpha == s.lora_alpha;
  for (const Entry& en : moe_entries(L)) {
    const int extra = file_lora && en.which != MOE_W_ROUTER ? 2 : 0;
    if (!en.mine) {   // an expert another rank owns
      if (!skip_params(in, s.precision, 1 + extra)) { L->err = "InvalidSnapshot: truncated weight file"; return MOE_INVALID_INPUT; }
      continue;
    }
    Tensor t;
    if ((rc = read_param(in, s.precision, en.rows, en.cols, &t, &L->err)) != MOE_OK) return rc;
    if ((rc = put_weight(L, en.which, en.expert, s.precision, t)) != MOE_OK) return rc;
    if (extra == 0) continue;
    if (!take_lora) {
      if (!skip_params(in, s.precision, 2)) { L->err = "InvalidSnapshot: truncated weight file"; return MOE_INVALID_INPUT; }
      continue;
    }
    Tensor down, up;
    if ((rc = read_param(in, s.precision, (uint64_t)s.lora_rank, en.cols, &down, &L->err)) != MOE_OK) return rc;
    if ((rc = read_param(in, s.precision, en.rows, (uint64_t)s.lora_rank, &up, &L->err)) != MOE_OK) return rc;
    for (Tensor* a : {&down, &up}) {
      if (s.precision != MOE_PRECISION_Q8) continue;
      a->f32.resize((size_t)(a->rows * a->cols));
      for (uint64_t r = 0; r < a->rows; ++r)
        for (uint64_t c = 0; c < a->cols; ++c)
          a->f32[(size_t)(r * a->cols + c)] = (float)a->q[(size_t)(r * a->cols + c)] * a->scale[(size_t)r];
    }
    if ((rc = moe_lora_set(L, en.which, en.expert, down.f32.data(), up.f32.data())) != MOE_OK) return rc;
  }
  return MOE_OK;
}

int32_t moe_load_optimizer_layer(moe_layer_t* L, const char* moments_path, const moe_snapshot_info_t* info,
                                 int32_t block_index, int64_t* step) {
  if (!L) return MOE_INVALID_INPUT;
  if (L->status != MOE_OK) return MOE_POISONED;
  if (!moments_path || !info) { L->err = "InvalidInput: null argument"; return MOE_INVALID_INPUT; }
  int rc = check_block(L, *info, block_index);
  if (rc != MOE_OK) return rc;
  if (info->lora_rank > 0) {
    L->err = "Unsupported: optimizer state of a model with LoRA adapters (the base weights are frozen, the adapter moments have no entry point yet)";
    return MOE_UNSUPPORTED;
  }
  File in(moments_path);
  char magic[8];
  uint64_t count = 0, file_step = 0;
  if (!in.f || !in.read(magic, 8) || memcmp(magic, "RBOPT001", 8) != 0) {
    L->err = "InvalidSnapshot: not a RustingBrain optimizer state file";   // transformer.rs:1706-1710
    return MOE_INVALID_INPUT;
  }
  if (!in.u64(&count) || !in.u64(&file_step)) { L->err = "InvalidSnapshot: truncated optimizer state file"; return MOE_INVALID_INPUT; }
  if ((int64_t)count != info->parameter_count) {
    L->err = "InvalidSnapshot: optimizer state holds " + std::to_string(count) + " parameters, this model has " +
             std::to_string(info->parameter_count);   // transformer.rs:1718-1723
    return MOE_INVALID_INPUT;
  }
  auto skip_moments = [&](int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
      uint64_t rows, cols;
      if (!in.u64(&rows) || !in.u64(&cols) || !in.skip(rows * cols * 8)) return false;
    }
    return true;
  };
  const Layout lay = layout_of(*info);
  if (!skip_moments(lay.ffn_first[(size_t)block_index])) { L->err = "InvalidSnapshot: truncated optimizer state file"; return MOE_INVALID_INPUT; }
  std::vector<float> m, v;
  for (const Entry& en : moe_entries(L)) {
    if (!en.mine) {
      if (!skip_moments(1)) { L->err = "InvalidSnapshot: truncated optimizer state file"; return MOE_INVALID_INPUT; }
      continue;
    }
    uint64_t rows, cols;
    if (!in.u64(&rows) || !in.u64(&cols)) { L->err = "InvalidSnapshot: truncated optimizer state file"; return MOE_INVALID_INPUT; }
    if (rows == 0 && cols == 0) continue;   // a frozen parameter released its moments (transformer.rs:1729-1735)
    if (rows != en.rows || cols != en.cols) {
      L->err = "InvalidSnapshot: optimizer state has a " + std::to_string(rows) + "x" + std::to_string(cols) +
               " parameter where the layer has " + std::to_string(en.rows) + "x" + std::to_string(en.cols);
      return MOE_INVALID_INPUT;
    }
    const size_t n = (size_t)(rows * cols);
    m.resize(n); v.resize(n);
    if (!in.read(m.data(), n * 4) || !in.read(v.data(), n * 4)) { L->err = "InvalidSnapshot: truncated optimizer state file"; return MOE_INVALID_INPUT; }
    if ((rc = moe_set_moments_f32(L, en.which, en.expert, m.data(), v.data(), (int32_t)rows, (int32_t)cols)) != MOE_OK) return rc;
  }
  if (step) *step = (int64_t)file_step;
  return MOE_OK;
}

int32_t moe_load_lora_layer(moe_layer_t* L, const char* lora_path, const moe_snapshot_info_t* info, int32_t block_index) {
  if (!L) return MOE_INVALID_INPUT;
  if (L->status != MOE_OK) return MOE_POISONED;
  if (!lora_path || !info) { L->err = "InvalidInput: null argument"; return MOE_INVALID_INPUT; }
  int rc = check_block(L, *info, block_index);
  if (rc != MOE_OK) return rc;
  if (L->lora_rank == 0) {   // transformer.rs:1168-1172
    L->err = "InvalidSnapshot: this layer has no LoRA adapter to load into; call moe_lora_attach first";
    return MOE_INVALID_INPUT;
  }
  File in(lora_path);
  char magic[8];
  uint64_t hlen = 0, count = 0;
  if (!in.f || !in.read(magic, 8) || memcmp(magic, "RBLOR001", 8) != 0) {
    L->err = "InvalidSnapshot: not a RustingBrain LoRA file";   // transformer.rs:1150-1154
    return MOE_INVALID_INPUT;
  }
  if (!in.u64(&hlen) || hlen == 0 || hlen > (1u << 20)) { L->err = "InvalidSnapshot: bad header length"; return MOE_INVALID_INPUT; }
  std::string text(hlen, '\0');
  if (!in.read(&text[0], hlen)) { L->err = "InvalidSnapshot: truncated header"; return MOE_INVALID_INPUT; }
  JsonParser jp{text.data(), text.data() + text.size()};
  const Json root = jp.value();
  const Json* jr = jp.ok ? root.get("rank") : nullptr;
  const Json* ja = jp.ok ? root.get("alpha") : nullptr;
  if (!jr || jr->kind != Json::Number || !ja || ja->kind != Json::Number) {
    L->err = "InvalidSnapshot: the header is not the LoraConfig save_lora writes";
    return MOE_INVALID_INPUT;
  }
  if ((int)jr->num != L->lora_rank || (float)ja->num != L->lora_alpha) {   // transformer.rs:1161-1167
    L->err = "InvalidSnapshot: adapter file holds rank " + std::to_string((int)jr->num) + " alpha " + std::to_string(ja->num) +
             ", this layer has rank " + std::to_string(L->lora_rank) + " alpha " + std::to_string(L->lora_alpha);
    return MOE_INVALID_INPUT;
  }
  // adapters sit on the four attention projections and on the feed-forward projections of every block
  // (transformer_block.rs:274-278; a MoE block: experts and shared expert, not the router), two
  // parameters each (down, up; param.rs:711-713), in block order
  auto linears_of = [&](int64_t b) {
    bool moe = false;
    for (int i = 0; i < info->n_moe_layers; ++i) moe = moe || info->moe_layers[i] == b;
    return (int64_t)4 + (moe ? 3 * info->num_experts + (info->shared_expert ? 3 : 0) : info->dense_ffn_params);
  };
  int64_t total = 0, before = 0;
  for (int64_t b = 0; b < info->n_layers; ++b) {
    if (b < block_index) before += linears_of(b);
    total += linears_of(b);
  }
  if (!in.u64(&count) || (int64_t)count != 2 * total) {   // transformer.rs:1178-1183
    L->err = "InvalidSnapshot: adapter file holds " + std::to_string(count) + " parameters, this model has " + std::to_string(2 * total);
    return MOE_INVALID_INPUT;
  }
  auto skip = [&](int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
      uint64_t rows, cols;
      if (!in.u64(&rows) || !in.u64(&cols) || !in.skip(rows * cols * 4)) return false;
    }
    return true;
  };
  auto read = [&](uint64_t want_rows, uint64_t want_cols, std::vector<float>* out) {
    uint64_t rows, cols;
    if (!in.u64(&rows) || !in.u64(&cols)) { L->err = "InvalidSnapshot: truncated adapter file"; return false; }
    if (rows != want_rows || cols != want_cols) {   // transformer.rs:1189-1194
      L->err = "InvalidSnapshot: adapter file has a " + std::to_string(rows) + "x" + std::to_string(cols) +
               " parameter where the layer has " + std::to_string(want_rows) + "x" + std::to_string(want_cols);
      return false;
    }
    out->resize((size_t)(rows * cols));
    if (!in.read(out->data(), out->size() * 4)) { L->err = "InvalidSnapshot: truncated adapter file"; return false; }
    return true;
  };
  if (!skip(2 * (before + 4))) { L->err = "InvalidSnapshot: truncated adapter file"; return MOE_INVALID_INPUT; }
  std::vector<float> down, up;
  for (const Entry& en : moe_entries(L)) {
    if (en.which == MOE_W_ROUTER) continue;
    if (!en.mine) {
      if (!skip(2)) { L->err = "InvalidSnapshot: truncated adapter file"; return MOE_INVALID_INPUT; }
      continue;
    }
    if (!read((uint64_t)L->lora_rank, en.cols, &down) || !read(en.rows, (uint64_t)L->lora_rank, &up)) return MOE_INVALID_INPUT;
    if ((rc = moe_lora_set(L, en.which, en.expert, down.data(), up.data())) != MOE_OK) return rc;
  }
  return MOE_OK;
}

}  // extern "C"
