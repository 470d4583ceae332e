// Checkpoints of a Sequential in the reference's file format (nn/models/serialization.v):
// save / save_checkpoint (:102-262), load_checkpoint (:266-276), load_weights (:279-373),
// encode_tensor / decode_tensor (:421-473).  The tensor payloads (f64 big-endian, base64) are
// produced and consumed on the device (vtlb_ckpt_encode_f32 / vtlb_ckpt_decode_f32); the host
// only frames them in JSON.  Optimizer moments, which the reference leaves out (its loader is
// commented out, :376-417), are written under that loader's key names.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>

#include "vtl_host.hpp"

namespace vtl {
namespace {

// ---------------------------------------------------------------- a small JSON reader
struct JValue {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<JValue> arr;
  std::vector<std::pair<std::string, JValue>> obj;  // insertion order kept
  const JValue* get(const std::string& key) const {
    for (const auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  const JValue& at(const std::string& key) const {
    const JValue* v = get(key);
    if (!v) throw Error(VTLB_EINVAL, "checkpoint: missing field '" + key + "'");
    return *v;
  }
};

class JParser {
 public:
  explicit JParser(const std::string& text) : s_(text) {}
  JValue parse() {
    JValue v = value();
    ws();
    if (p_ != s_.size()) fail("trailing characters");
    return v;
  }

 private:
  const std::string& s_;
  size_t p_ = 0;
  int depth_ = 0;  // nesting of the value being read; a checkpoint has five levels
  struct Nest {
    JParser& p;
    explicit Nest(JParser& parser) : p(parser) {
      if (++p.depth_ > 64) p.fail("nested too deeply");
    }
    ~Nest() { --p.depth_; }
  };
  [[noreturn]] void fail(const char* what) const {
    throw Error(VTLB_EINVAL, std::string("checkpoint: malformed JSON (") + what + " at byte " + std::to_string(p_) + ")");
  }
  void ws() {
    while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) ++p_;
  }
  bool eat(char c) {
    ws();
    if (p_ < s_.size() && s_[p_] == c) {
      ++p_;
      return true;
    }
    return false;
  }
  std::string string_body() {
    std::string out;
    // a payload of 134 M parameters is one 1.4 GB string: copy unescaped runs in one piece
    for (;;) {
      const size_t q = s_.find_first_of("\"\\", p_);
      if (q == std::string::npos) fail("unterminated string");
      out.append(s_, p_, q - p_);
      p_ = q;
      if (s_[p_] == '"') {
        ++p_;
        return out;
      }
      if (p_ + 1 >= s_.size()) fail("bad escape");
      const char e = s_[p_ + 1];
      p_ += 2;
      switch (e) {
        case '"': out += '"'; break;
        case '\\': out += '\\'; break;
        case '/': out += '/'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'n': out += '\n'; break;
        case 'r': out += '\r'; break;
        case 't': out += '\t'; break;
        case 'u': {
          if (p_ + 4 > s_.size()) fail("bad \\u escape");
          const unsigned cp = (unsigned)std::strtoul(s_.substr(p_, 4).c_str(), nullptr, 16);
          p_ += 4;
          if (cp < 0x80) {
            out += (char)cp;
          } else if (cp < 0x800) {
            out += (char)(0xC0 | (cp >> 6));
            out += (char)(0x80 | (cp & 0x3F));
          } else {
            out += (char)(0xE0 | (cp >> 12));
            out += (char)(0x80 | ((cp >> 6) & 0x3F));
            out += (char)(0x80 | (cp & 0x3F));
          }
          break;
        }
        default: fail("bad escape");
      }
    }
  }
  JValue value() {
    ws();
    if (p_ >= s_.size()) fail("unexpected end");
    const Nest nest(*this);
    JValue v;
    const char c = s_[p_];
    if (c == '{') {
      ++p_;
      v.kind = JValue::Obj;
      if (eat('}')) return v;
      do {
        ws();
        if (p_ >= s_.size() || s_[p_] != '"') fail("object key expected");
        ++p_;
        std::string key = string_body();
        if (!eat(':')) fail("':' expected");
        v.obj.emplace_back(std::move(key), value());
      } while (eat(','));
      if (!eat('}')) fail("'}' expected");
    } else if (c == '[') {
      ++p_;
      v.kind = JValue::Arr;
      if (eat(']')) return v;
      do v.arr.push_back(value());
      while (eat(','));
      if (!eat(']')) fail("']' expected");
    } else if (c == '"') {
      ++p_;
      v.kind = JValue::Str;
      v.str = string_body();
    } else if (!s_.compare(p_, 4, "true")) {
      p_ += 4;
      v.kind = JValue::Bool;
      v.b = true;
    } else if (!s_.compare(p_, 5, "false")) {
      p_ += 5;
      v.kind = JValue::Bool;
    } else if (!s_.compare(p_, 4, "null")) {
      p_ += 4;
    } else {
      // a JSON number and nothing else: -? int frac? exp?  (strtod alone would also take
      // "nan", "inf" and hexadecimal floats, which a JSON decoder rejects)
      size_t q = p_;
      auto digits = [&] {
        const size_t q0 = q;
        while (q < s_.size() && s_[q] >= '0' && s_[q] <= '9') ++q;
        return q > q0;
      };
      if (q < s_.size() && s_[q] == '-') ++q;
      if (!digits()) fail("value expected");
      if (q < s_.size() && s_[q] == '.') {
        ++q;
        if (!digits()) fail("digits expected after the decimal point");
      }
      if (q < s_.size() && (s_[q] == 'e' || s_[q] == 'E')) {
        ++q;
        if (q < s_.size() && (s_[q] == '+' || s_[q] == '-')) ++q;
        if (!digits()) fail("digits expected in the exponent");
      }
      v.num = std::strtod(s_.substr(p_, q - p_).c_str(), nullptr);
      p_ = q;
      v.kind = JValue::Num;
    }
    return v;
  }
};

std::string read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw Error(VTLB_EINVAL, "checkpoint: cannot open '" + path + "'");
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

void json_string(std::string& out, const std::string& s) {
  out += '"';
  for (char c : s) {
    if (c == '"' || c == '\\') {
      out += '\\';
      out += c;
    } else if ((unsigned char)c < 0x20) {
      char buf[8];
      std::snprintf(buf, sizeof buf, "\\u%04x", c);
      out += buf;
    } else {
      out += c;
    }
  }
  out += '"';
}
std::string json_number(double v) {
  if (!(v - v == 0.0)) return "null";  // JSON has no NaN or infinity
  char buf[40];
  std::snprintf(buf, sizeof buf, "%.17g", v);
  return buf;
}
std::string shape_list(const std::vector<int>& shape, const char* sep) {
  std::string s;
  for (size_t i = 0; i < shape.size(); ++i) {
    if (i) s += sep;
    s += std::to_string(shape[i]);
  }
  return s;
}

// "<shape>;row_major|<base64 of the f64 big-endian bytes>" (encode_tensor, serialization.v:421-438)
std::string encode_tensor(const Tensor& t) {
  Session* s = t.session();
  const size_t n = t.size(), len = vtlb_ckpt_text_len(n);
  std::string out = shape_list(t.shape(), ",") + ";row_major|";
  if (n == 0) return out;
  void* d_text = nullptr;
  s->check(vtlb_alloc(s->ctx, len, &d_text));
  int rc = vtlb_ckpt_encode_f32(s->ctx, t.data(), n, d_text);
  const size_t head = out.size();
  out.resize(head + len);
  if (rc == VTLB_OK) rc = vtlb_d2h(s->ctx, &out[head], d_text, len);
  vtlb_free(s->ctx, d_text);
  s->check(rc);
  return out;
}

// decode_tensor (serialization.v:441-473) into an existing device tensor
void decode_tensor_into(const std::string& encoded, const Tensor& dst) {
  const size_t bar = encoded.find('|');
  if (bar == std::string::npos || encoded.find('|', bar + 1) != std::string::npos)
    throw Error(VTLB_EINVAL, "Invalid tensor encoding: missing shape delimiter");
  const std::string head = encoded.substr(0, bar);
  const std::string shape_str = head.substr(0, head.find(';'));
  std::vector<int> decoded_shape;
  {
    std::stringstream ss(shape_str);
    std::string item;
    while (std::getline(ss, item, ',')) decoded_shape.push_back(std::atoi(item.c_str()));
  }
  if (decoded_shape != dst.shape())
    throw Error(VTLB_EINVAL, "Shape mismatch: encoded [" + shape_list(decoded_shape, ", ") + "], expected [" +
                                 shape_list(dst.shape(), ", ") + "]");
  Session* s = dst.session();
  const size_t n = dst.size(), len = encoded.size() - bar - 1;
  if (n == 0) return;
  if (len != vtlb_ckpt_text_len(n))
    throw Error(VTLB_EINVAL, "Invalid tensor encoding: " + std::to_string(len) + " characters for " +
                                 std::to_string(n) + " values");
  void* d_text = nullptr;
  s->check(vtlb_alloc(s->ctx, len, &d_text));
  int rc = vtlb_h2d(s->ctx, d_text, encoded.data() + bar + 1, len);
  if (rc == VTLB_OK) rc = vtlb_ckpt_decode_f32(s->ctx, d_text, len, dst.data(), n);
  vtlb_free(s->ctx, d_text);
  s->check(rc);
}

const char* weight_key(const std::string& layer_type, size_t j, std::string& scratch) {
  if (layer_type == "LinearLayer" || layer_type == "Conv2DLayer") return j == 0 ? "weight" : "bias";
  if (layer_type == "BatchNorm1DLayer" && j < 2) return j == 0 ? "gamma" : "beta";
  scratch = "var_" + std::to_string(j);
  return scratch.c_str();
}

JValue parse_model(const std::string& path) {
  const std::string text = read_file(path);
  JValue model = JParser(text).parse();
  if (model.kind != JValue::Obj) throw Error(VTLB_EINVAL, "checkpoint: top level is not an object");
  const std::string version = model.at("version").str;
  if (version != "1.0") throw Error(VTLB_EINVAL, "Model version mismatch: expected 1.0, got " + version);
  return model;
}

}  // namespace

// ---------------------------------------------------------------- Sequential
void Sequential::save(const std::string& path) { save_checkpoint(path, 0, 0.0, nullptr); }

void Sequential::save_checkpoint(const std::string& path, int epoch, double loss, const AdamOptimizer* opt) {
  std::string layer_defs = "[", layer_data = "[";
  for (size_t i = 0; i < layers.size(); ++i) {
    Layer* l = layers[i].get();
    const std::string type = l->type_name();
    if (i) {
      layer_defs += ',';
      layer_data += ',';
    }
    layer_defs += "{\"layer_type\":";
    json_string(layer_defs, type);
    layer_defs += ",\"in_shape\":[" + (i ? shape_list(layers[i - 1]->output_shape(), ",") : std::string()) + "],\"config\":{";
    bool first = true;
    for (const auto& kv : l->config()) {
      if (!first) layer_defs += ',';
      first = false;
      json_string(layer_defs, kv.first);
      layer_defs += ':' + std::to_string(kv.second);
    }
    layer_defs += "}}";
    layer_data += "{\"weights\":{";
    const auto vars = l->variables();
    for (size_t j = 0; j < vars.size(); ++j) {
      std::string scratch;
      if (j) layer_data += ',';
      json_string(layer_data, weight_key(type, j, scratch));
      layer_data += ':';
      json_string(layer_data, encode_tensor(vars[j]->value));
    }
    layer_data += "}}";
  }
  layer_defs += ']';
  layer_data += ']';

  std::string optimizer = "{\"optimizer_type\":\"\",\"learning_rate\":0,\"config\":{},\"moments\":{}}";
  if (opt) {
    optimizer = std::string("{\"optimizer_type\":\"") + (opt->adamw ? "AdamWOptimizer" : "AdamOptimizer") +
                "\",\"learning_rate\":" + json_number(opt->learning_rate) + ",\"config\":{\"beta1\":" +
                json_number(opt->beta1) + ",\"beta2\":" + json_number(opt->beta2) + ",\"epsilon\":" +
                json_number(opt->epsilon) + ",\"weight_decay\":" + json_number(opt->weight_decay) +
                ",\"beta1_t\":" + json_number(opt->beta1_t) + ",\"beta2_t\":" + json_number(opt->beta2_t) +
                "},\"moments\":{";
    for (size_t i = 0; i < opt->params.size(); ++i) {
      if (i) optimizer += ',';
      optimizer += "\"moment_" + std::to_string(i) + "\":";
      json_string(optimizer, encode_tensor(opt->first_moments[i]));
      optimizer += ",\"second_moment_" + std::to_string(i) + "\":";
      json_string(optimizer, encode_tensor(opt->second_moments[i]));
    }
    optimizer += "}}";
  }

  // Written beside the target and renamed over it once it is complete and closed, so that a
  // failure half way (disk full, process killed) leaves the previous checkpoint untouched.
  const std::string tmp = path + ".tmp";
  {
    std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
    if (!f) throw Error(VTLB_EINVAL, "checkpoint: cannot write '" + path + "'");
    f << "{\"version\":\"1.0\",\"layers\":" << layer_defs << ",\"layer_data\":" << layer_data
      << ",\"optimizer\":" << optimizer << ",\"metadata\":{\"epoch\":" << epoch << ",\"loss\":" << json_number(loss)
      << ",\"saved_at\":\"vtl_checkpoint\",\"version\":\"1.0\"}}";
    f.flush();
    f.close();
    if (f.fail()) {
      std::remove(tmp.c_str());
      throw Error(VTLB_EINVAL, "checkpoint: write to '" + path + "' failed");
    }
  }
  if (std::rename(tmp.c_str(), path.c_str()) != 0) {
    std::remove(tmp.c_str());
    throw Error(VTLB_EINVAL, "checkpoint: cannot replace '" + path + "'");
  }
}

std::pair<int, double> Sequential::load_checkpoint(const std::string& path) {
  const JValue model = parse_model(path);
  const JValue& meta = model.at("metadata");
  return {(int)meta.at("epoch").num, meta.at("loss").num};
}

void Sequential::load_weights(const std::string& path, AdamOptimizer* opt) {
  const JValue model = parse_model(path);
  const JValue& defs = model.at("layers");
  const JValue& data = model.at("layer_data");
  if (defs.arr.size() != layers.size())
    throw Error(VTLB_EINVAL, "Layer count mismatch: model has " + std::to_string(layers.size()) + ", checkpoint has " +
                                 std::to_string(defs.arr.size()));
  if (data.arr.size() != defs.arr.size()) throw Error(VTLB_EINVAL, "checkpoint: layer_data and layers differ in length");
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string saved_type = defs.arr[i].at("layer_type").str;
    const std::string current_type = layers[i]->type_name();
    if (saved_type != current_type)
      throw Error(VTLB_EINVAL, "Layer " + std::to_string(i) + " type mismatch: expected " + saved_type + ", got " + current_type);
    const JValue& weights = data.arr[i].at("weights");
    const auto vars = layers[i]->variables();
    for (size_t j = 0; j < vars.size(); ++j) {
      std::string scratch;
      const std::string key = weight_key(saved_type, j, scratch);
      const JValue* enc = weights.get(key);
      if (!enc) throw Error(VTLB_EINVAL, "Missing weight " + key + " for layer " + std::to_string(i));
      decode_tensor_into(enc->str, vars[j]->value);
    }
  }
  if (opt) {
    const JValue& o = model.at("optimizer");
    const JValue& moments = o.at("moments");
    if (moments.obj.empty()) throw Error(VTLB_EINVAL, "checkpoint: no optimizer moments stored");
    const std::string want = opt->adamw ? "AdamWOptimizer" : "AdamOptimizer";
    if (o.at("optimizer_type").str != want)
      throw Error(VTLB_EINVAL, "Optimizer type mismatch: expected " + want + ", got " + o.at("optimizer_type").str);
    const JValue& cfg = o.at("config");
    if (const JValue* v = cfg.get("beta1_t")) opt->beta1_t = v->num;
    if (const JValue* v = cfg.get("beta2_t")) opt->beta2_t = v->num;
    for (size_t i = 0; i < opt->params.size(); ++i) {
      const JValue* m = moments.get("moment_" + std::to_string(i));
      const JValue* v = moments.get("second_moment_" + std::to_string(i));
      if (!m || !v) throw Error(VTLB_EINVAL, "Missing optimizer moment " + std::to_string(i));
      decode_tensor_into(m->str, opt->first_moments[i]);
      decode_tensor_into(v->str, opt->second_moments[i]);
    }
  }
}

}  // namespace vtl
