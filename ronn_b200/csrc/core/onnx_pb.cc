// ONNX protobuf wire-format decoder and encoder.
//
// Replaces the reference's prost-generated decoder
// (crates/ronn-onnx/build.rs:3-16, crates/ronn-onnx/src/loader.rs:22-154) with a
// hand-written schema-aware reader that never copies tensor payloads: every
// initializer is reported as an (offset, length) window into the caller's
// buffer (raw_data) or as a freshly packed little-endian blob (typed fields).
//
// Decoding produces a compact JSON description of the model (graph structure,
// attributes, value infos, tensor descriptors) that the Python layer turns into
// the graph IR; payload bytes stay where they are.  Encoding is a small
// builder API (begin -> add_* -> finish) used by the model writers.
//
// All entry points are extern "C" so they can be reached through ctypes.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include <memory>
#include <stdexcept>
#include <limits>

namespace {

struct ParseError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// ---------------------------------------------------------------- wire reader
struct Reader {
  const uint8_t* base;   // start of the whole model buffer (for offsets)
  const uint8_t* p;
  const uint8_t* end;
  int depth;

  bool done() const { return p >= end; }

  uint64_t varint() {
    uint64_t v = 0;
    int shift = 0;
    while (true) {
      if (p >= end) throw ParseError("truncated varint");
      uint8_t b = *p++;
      if (shift < 64) v |= uint64_t(b & 0x7f) << shift;
      if (!(b & 0x80)) break;
      shift += 7;
      if (shift > 70) throw ParseError("varint too long");
    }
    return v;
  }
  uint32_t fixed32() {
    if (end - p < 4) throw ParseError("truncated fixed32");
    uint32_t v;
    memcpy(&v, p, 4);
    p += 4;
    return v;
  }
  uint64_t fixed64() {
    if (end - p < 8) throw ParseError("truncated fixed64");
    uint64_t v;
    memcpy(&v, p, 8);
    p += 8;
    return v;
  }
  Reader sub() {
    uint64_t n = varint();
    if (n > uint64_t(end - p)) throw ParseError("length-delimited field overruns buffer");
    if (depth > 64) throw ParseError("message nesting too deep");
    Reader r{base, p, p + n, depth + 1};
    p += n;
    return r;
  }
  std::string str() {
    Reader r = sub();
    return std::string(reinterpret_cast<const char*>(r.p), size_t(r.end - r.p));
  }
  void skip(uint32_t wt) {
    switch (wt) {
      case 0: varint(); break;
      case 1: fixed64(); break;
      case 2: sub(); break;
      case 5: fixed32(); break;
      default: throw ParseError("unsupported wire type " + std::to_string(wt));
    }
  }
  // returns false at end of message
  bool tag(uint32_t& field, uint32_t& wt) {
    if (p >= end) return false;
    uint64_t t = varint();
    field = uint32_t(t >> 3);
    wt = uint32_t(t & 7);
    if (field == 0) throw ParseError("field number 0");
    return true;
  }
};

// ---------------------------------------------------------------- JSON writer
struct Json {
  std::string s;
  void raw(const char* c) { s += c; }
  void str(const std::string& v) {
    s.push_back('"');
    for (unsigned char c : v) {
      switch (c) {
        case '"': s += "\\\""; break;
        case '\\': s += "\\\\"; break;
        case '\n': s += "\\n"; break;
        case '\r': s += "\\r"; break;
        case '\t': s += "\\t"; break;
        default:
          if (c < 0x20 || c >= 0x7f) {
            // bytes outside printable ASCII are carried as \u00XX; Python
            // re-assembles them as latin-1 and re-decodes as UTF-8.
            char buf[8];
            snprintf(buf, sizeof buf, "\\u%04x", c);
            s += buf;
          } else {
            s.push_back(char(c));
          }
      }
    }
    s.push_back('"');
  }
  void i64(int64_t v) { s += std::to_string(v); }
  void u64(uint64_t v) { s += std::to_string(v); }
  void f32(float v) {
    if (v != v) { s += "\"nan\""; return; }
    if (v == std::numeric_limits<float>::infinity()) { s += "\"inf\""; return; }
    if (v == -std::numeric_limits<float>::infinity()) { s += "\"-inf\""; return; }
    char buf[40];
    snprintf(buf, sizeof buf, "%.9g", double(v));
    s += buf;
  }
};

// ---------------------------------------------------------------- model structs
struct TensorDesc {
  std::string name;
  std::vector<int64_t> dims;
  int32_t data_type = 0;
  // payload: either a window into the source buffer or an owned blob index
  int64_t raw_off = -1, raw_len = 0;
  int64_t blob = -1;
  bool external = false;
  std::vector<std::pair<std::string, std::string>> external_data;
  // typed repeated fields gathered during parsing
  std::vector<float> f32s;
  std::vector<int32_t> i32s;
  std::vector<int64_t> i64s;
  std::vector<double> f64s;
  std::vector<uint64_t> u64s;
  std::vector<std::string> strs;
};

struct Parsed {
  std::string json;
  std::vector<std::vector<uint8_t>> blobs;
  std::string error;
};

template <class T, class F>
void packed_or_single(Reader& r, uint32_t wt, std::vector<T>& out, F readone, uint32_t single_wt) {
  if (wt == 2) {
    Reader s = r.sub();
    while (!s.done()) out.push_back(readone(s));
  } else if (wt == single_wt) {
    out.push_back(readone(r));
  } else {
    throw ParseError("bad wire type for repeated scalar");
  }
}

float rd_f32(Reader& r) { uint32_t u = r.fixed32(); float f; memcpy(&f, &u, 4); return f; }
double rd_f64(Reader& r) { uint64_t u = r.fixed64(); double f; memcpy(&f, &u, 8); return f; }
int64_t rd_i64(Reader& r) { return int64_t(r.varint()); }
int32_t rd_i32(Reader& r) { return int32_t(int64_t(r.varint())); }
uint64_t rd_u64(Reader& r) { return r.varint(); }

void parse_kv(Reader r, std::string& k, std::string& v) {
  uint32_t f, wt;
  while (r.tag(f, wt)) {
    if (f == 1 && wt == 2) k = r.str();
    else if (f == 2 && wt == 2) v = r.str();
    else r.skip(wt);
  }
}

int elem_size(int32_t dt) {
  switch (dt) {
    case 1: return 4;   // FLOAT
    case 2: return 1;   // UINT8
    case 3: return 1;   // INT8
    case 4: return 2;   // UINT16
    case 5: return 2;   // INT16
    case 6: return 4;   // INT32
    case 7: return 8;   // INT64
    case 9: return 1;   // BOOL
    case 10: return 2;  // FLOAT16
    case 11: return 8;  // DOUBLE
    case 12: return 4;  // UINT32
    case 13: return 8;  // UINT64
    case 16: return 2;  // BFLOAT16
    case 17: case 18: case 19: case 20: return 1;  // FLOAT8*
    default: return 0;
  }
}

TensorDesc parse_tensor(Reader r, Parsed& out) {
  TensorDesc t;
  uint32_t f, wt;
  int64_t data_location = 0;
  while (r.tag(f, wt)) {
    switch (f) {
      case 1: packed_or_single(r, wt, t.dims, rd_i64, 0); break;
      case 2: if (wt != 0) throw ParseError("tensor data_type wire type"); t.data_type = int32_t(r.varint()); break;
      case 4: packed_or_single(r, wt, t.f32s, rd_f32, 5); break;
      case 5: packed_or_single(r, wt, t.i32s, rd_i32, 0); break;
      case 6: if (wt != 2) throw ParseError("string_data wire type"); t.strs.push_back(r.str()); break;
      case 7: packed_or_single(r, wt, t.i64s, rd_i64, 0); break;
      case 8: if (wt != 2) throw ParseError("tensor name wire type"); t.name = r.str(); break;
      case 9: {
        if (wt != 2) throw ParseError("raw_data wire type");
        Reader s = r.sub();
        t.raw_off = int64_t(s.p - s.base);
        t.raw_len = int64_t(s.end - s.p);
        break;
      }
      case 10: packed_or_single(r, wt, t.f64s, rd_f64, 1); break;
      case 11: packed_or_single(r, wt, t.u64s, rd_u64, 0); break;
      case 13: {
        if (wt != 2) throw ParseError("external_data wire type");
        std::string k, v;
        parse_kv(r.sub(), k, v);
        t.external_data.emplace_back(k, v);
        break;
      }
      case 14: if (wt != 0) throw ParseError("data_location wire type"); data_location = int64_t(r.varint()); break;
      default: r.skip(wt);
    }
  }
  t.external = (data_location == 1);
  // Typed fields -> packed little-endian blob in the tensor's own element type.
  if (t.raw_off < 0 && !t.external) {
    std::vector<uint8_t> blob;
    auto put = [&blob](const void* p, size_t n) {
      const uint8_t* b = static_cast<const uint8_t*>(p);
      blob.insert(blob.end(), b, b + n);
    };
    switch (t.data_type) {
      case 1: for (float v : t.f32s) put(&v, 4); break;
      case 11: for (double v : t.f64s) put(&v, 8); break;
      case 7: for (int64_t v : t.i64s) put(&v, 8); break;
      case 13: for (uint64_t v : t.u64s) put(&v, 8); break;
      case 12: for (uint64_t v : t.u64s) { uint32_t w = uint32_t(v); put(&w, 4); } break;
      case 6: for (int32_t v : t.i32s) put(&v, 4); break;
      case 2: case 3: case 9: case 17: case 18: case 19: case 20:
        for (int32_t v : t.i32s) { uint8_t w = uint8_t(v); put(&w, 1); } break;
      case 4: case 5: case 10: case 16:
        for (int32_t v : t.i32s) { uint16_t w = uint16_t(v); put(&w, 2); } break;
      default: break;
    }
    if (!blob.empty()) {
      t.blob = int64_t(out.blobs.size());
      out.blobs.push_back(std::move(blob));
    }
  }
  return t;
}

void emit_tensor(Json& j, const TensorDesc& t) {
  j.raw("{\"name\":"); j.str(t.name);
  j.raw(",\"dims\":[");
  for (size_t i = 0; i < t.dims.size(); ++i) { if (i) j.raw(","); j.i64(t.dims[i]); }
  j.raw("],\"data_type\":"); j.i64(t.data_type);
  j.raw(",\"raw_off\":"); j.i64(t.raw_off);
  j.raw(",\"raw_len\":"); j.i64(t.raw_len);
  j.raw(",\"blob\":"); j.i64(t.blob);
  j.raw(",\"external\":"); j.raw(t.external ? "true" : "false");
  if (!t.external_data.empty()) {
    j.raw(",\"external_data\":{");
    for (size_t i = 0; i < t.external_data.size(); ++i) {
      if (i) j.raw(",");
      j.str(t.external_data[i].first); j.raw(":"); j.str(t.external_data[i].second);
    }
    j.raw("}");
  }
  if (!t.strs.empty()) {
    j.raw(",\"strings\":[");
    for (size_t i = 0; i < t.strs.size(); ++i) { if (i) j.raw(","); j.str(t.strs[i]); }
    j.raw("]");
  }
  j.raw("}");
}

void parse_value_info(Reader r, Json& j) {
  std::string name;
  int64_t elem_type = 0;
  bool has_shape = false;
  std::string dims_json;
  uint32_t f, wt;
  while (r.tag(f, wt)) {
    if (f == 1 && wt == 2) name = r.str();
    else if (f == 2 && wt == 2) {
      Reader tp = r.sub();
      uint32_t f2, wt2;
      while (tp.tag(f2, wt2)) {
        if (f2 == 1 && wt2 == 2) {  // tensor_type
          Reader tt = tp.sub();
          uint32_t f3, wt3;
          while (tt.tag(f3, wt3)) {
            if (f3 == 1 && wt3 == 0) elem_type = int64_t(tt.varint());
            else if (f3 == 2 && wt3 == 2) {
              has_shape = true;
              Reader sh = tt.sub();
              uint32_t f4, wt4;
              Json dj;
              bool first = true;
              while (sh.tag(f4, wt4)) {
                if (f4 == 1 && wt4 == 2) {
                  Reader d = sh.sub();
                  uint32_t f5, wt5;
                  bool has_val = false; int64_t val = 0; std::string param;
                  while (d.tag(f5, wt5)) {
                    if (f5 == 1 && wt5 == 0) { val = int64_t(d.varint()); has_val = true; }
                    else if (f5 == 2 && wt5 == 2) param = d.str();
                    else d.skip(wt5);
                  }
                  if (!first) dj.raw(",");
                  first = false;
                  if (has_val) dj.i64(val);
                  else dj.str(param);
                } else sh.skip(wt4);
              }
              dims_json = dj.s;
            } else tt.skip(wt3);
          }
        } else tp.skip(wt2);
      }
    } else r.skip(wt);
  }
  j.raw("{\"name\":"); j.str(name);
  j.raw(",\"elem_type\":"); j.i64(elem_type);
  if (has_shape) { j.raw(",\"shape\":["); j.s += dims_json; j.raw("]"); }
  else j.raw(",\"shape\":null");
  j.raw("}");
}

void parse_graph(Reader r, Json& j, Parsed& out);

void parse_attribute(Reader r, Json& j, Parsed& out) {
  std::string name, s_val, ref_attr;
  bool has_f = false, has_i = false, has_s = false, has_t = false, has_g = false;
  float fv = 0; int64_t iv = 0; int64_t type = 0;
  std::vector<float> floats; std::vector<int64_t> ints; std::vector<std::string> strings;
  TensorDesc tv; std::string graph_json;
  std::vector<TensorDesc> tensors;
  uint32_t f, wt;
  while (r.tag(f, wt)) {
    switch (f) {
      case 1: if (wt != 2) throw ParseError("attr name"); name = r.str(); break;
      case 2: if (wt != 5) throw ParseError("attr f"); fv = rd_f32(r); has_f = true; break;
      case 3: if (wt != 0) throw ParseError("attr i"); iv = int64_t(r.varint()); has_i = true; break;
      case 4: if (wt != 2) throw ParseError("attr s"); s_val = r.str(); has_s = true; break;
      case 5: if (wt != 2) throw ParseError("attr t"); tv = parse_tensor(r.sub(), out); has_t = true; break;
      case 6: { if (wt != 2) throw ParseError("attr g"); Json g; parse_graph(r.sub(), g, out); graph_json = g.s; has_g = true; break; }
      case 7: packed_or_single(r, wt, floats, rd_f32, 5); break;
      case 8: packed_or_single(r, wt, ints, rd_i64, 0); break;
      case 9: if (wt != 2) throw ParseError("attr strings"); strings.push_back(r.str()); break;
      case 10: if (wt != 2) throw ParseError("attr tensors"); tensors.push_back(parse_tensor(r.sub(), out)); break;
      case 20: if (wt != 0) throw ParseError("attr type"); type = int64_t(r.varint()); break;
      case 21: if (wt != 2) throw ParseError("attr ref"); ref_attr = r.str(); break;
      default: r.skip(wt);
    }
  }
  // Infer the type when the producer did not set it (old exporters).
  if (type == 0) {
    if (has_f) type = 1; else if (has_i) type = 2; else if (has_s) type = 3;
    else if (has_t) type = 4; else if (has_g) type = 5; else if (!floats.empty()) type = 6;
    else if (!ints.empty()) type = 7; else if (!strings.empty()) type = 8;
    else if (!tensors.empty()) type = 9;
  }
  j.raw("{\"name\":"); j.str(name); j.raw(",\"type\":"); j.i64(type);
  switch (type) {
    case 1: j.raw(",\"f\":"); j.f32(fv); break;
    case 2: j.raw(",\"i\":"); j.i64(iv); break;
    case 3: j.raw(",\"s\":"); j.str(s_val); break;
    case 4: j.raw(",\"t\":"); emit_tensor(j, tv); break;
    case 5: j.raw(",\"g\":"); j.s += graph_json.empty() ? "null" : graph_json; break;
    case 6: j.raw(",\"floats\":["); for (size_t i = 0; i < floats.size(); ++i) { if (i) j.raw(","); j.f32(floats[i]); } j.raw("]"); break;
    case 7: j.raw(",\"ints\":["); for (size_t i = 0; i < ints.size(); ++i) { if (i) j.raw(","); j.i64(ints[i]); } j.raw("]"); break;
    case 8: j.raw(",\"strings\":["); for (size_t i = 0; i < strings.size(); ++i) { if (i) j.raw(","); j.str(strings[i]); } j.raw("]"); break;
    case 9: j.raw(",\"tensors\":["); for (size_t i = 0; i < tensors.size(); ++i) { if (i) j.raw(","); emit_tensor(j, tensors[i]); } j.raw("]"); break;
    default: break;
  }
  if (!ref_attr.empty()) { j.raw(",\"ref_attr_name\":"); j.str(ref_attr); }
  j.raw("}");
}

void parse_node(Reader r, Json& j, Parsed& out) {
  std::vector<std::string> inputs, outputs;
  std::string name, op_type, domain;
  Json attrs;
  bool first_attr = true;
  uint32_t f, wt;
  while (r.tag(f, wt)) {
    switch (f) {
      case 1: if (wt != 2) throw ParseError("node input"); inputs.push_back(r.str()); break;
      case 2: if (wt != 2) throw ParseError("node output"); outputs.push_back(r.str()); break;
      case 3: if (wt != 2) throw ParseError("node name"); name = r.str(); break;
      case 4: if (wt != 2) throw ParseError("node op_type"); op_type = r.str(); break;
      case 5: {
        if (wt != 2) throw ParseError("node attribute");
        if (!first_attr) attrs.raw(",");
        first_attr = false;
        parse_attribute(r.sub(), attrs, out);
        break;
      }
      case 7: if (wt != 2) throw ParseError("node domain"); domain = r.str(); break;
      default: r.skip(wt);
    }
  }
  j.raw("{\"name\":"); j.str(name);
  j.raw(",\"op_type\":"); j.str(op_type);
  j.raw(",\"domain\":"); j.str(domain);
  j.raw(",\"inputs\":[");
  for (size_t i = 0; i < inputs.size(); ++i) { if (i) j.raw(","); j.str(inputs[i]); }
  j.raw("],\"outputs\":[");
  for (size_t i = 0; i < outputs.size(); ++i) { if (i) j.raw(","); j.str(outputs[i]); }
  j.raw("],\"attributes\":["); j.s += attrs.s; j.raw("]}");
}

void parse_graph(Reader r, Json& j, Parsed& out) {
  Json nodes, inits, inputs, outputs, vinfo;
  bool fn = true, fi = true, fin = true, fo = true, fv = true;
  std::string name, doc;
  uint32_t f, wt;
  while (r.tag(f, wt)) {
    switch (f) {
      case 1: if (wt != 2) throw ParseError("graph node"); if (!fn) nodes.raw(","); fn = false; parse_node(r.sub(), nodes, out); break;
      case 2: if (wt != 2) throw ParseError("graph name"); name = r.str(); break;
      case 5: {
        if (wt != 2) throw ParseError("graph initializer");
        if (!fi) inits.raw(",");
        fi = false;
        TensorDesc t = parse_tensor(r.sub(), out);
        emit_tensor(inits, t);
        break;
      }
      case 10: if (wt != 2) throw ParseError("graph doc"); doc = r.str(); break;
      case 11: if (wt != 2) throw ParseError("graph input"); if (!fin) inputs.raw(","); fin = false; parse_value_info(r.sub(), inputs); break;
      case 12: if (wt != 2) throw ParseError("graph output"); if (!fo) outputs.raw(","); fo = false; parse_value_info(r.sub(), outputs); break;
      case 13: if (wt != 2) throw ParseError("graph value_info"); if (!fv) vinfo.raw(","); fv = false; parse_value_info(r.sub(), vinfo); break;
      case 15: throw ParseError("sparse initializers are not supported");
      default: r.skip(wt);
    }
  }
  j.raw("{\"name\":"); j.str(name);
  j.raw(",\"doc_string\":"); j.str(doc);
  j.raw(",\"nodes\":["); j.s += nodes.s;
  j.raw("],\"initializers\":["); j.s += inits.s;
  j.raw("],\"inputs\":["); j.s += inputs.s;
  j.raw("],\"outputs\":["); j.s += outputs.s;
  j.raw("],\"value_info\":["); j.s += vinfo.s;
  j.raw("]}");
}

void parse_model(const uint8_t* data, size_t n, Parsed& out) {
  Reader r{data, data, data + n, 0};
  Json j;
  int64_t ir_version = 0, model_version = 0;
  bool has_ir = false, has_graph = false;
  std::string producer_name, producer_version, domain, doc, graph_json;
  Json opsets, meta;
  bool fo = true, fm = true;
  uint32_t f, wt;
  while (r.tag(f, wt)) {
    switch (f) {
      case 1: if (wt != 0) throw ParseError("ir_version wire type"); ir_version = int64_t(r.varint()); has_ir = true; break;
      case 2: if (wt != 2) throw ParseError("producer_name wire type"); producer_name = r.str(); break;
      case 3: if (wt != 2) throw ParseError("producer_version wire type"); producer_version = r.str(); break;
      case 4: if (wt != 2) throw ParseError("domain wire type"); domain = r.str(); break;
      case 5: if (wt != 0) throw ParseError("model_version wire type"); model_version = int64_t(r.varint()); break;
      case 6: if (wt != 2) throw ParseError("doc_string wire type"); doc = r.str(); break;
      case 7: {
        if (wt != 2) throw ParseError("graph wire type");
        Json g;
        parse_graph(r.sub(), g, out);
        graph_json = g.s;
        has_graph = true;
        break;
      }
      case 8: {
        if (wt != 2) throw ParseError("opset_import wire type");
        Reader s = r.sub();
        std::string d; int64_t v = 0;
        uint32_t f2, wt2;
        while (s.tag(f2, wt2)) {
          if (f2 == 1 && wt2 == 2) d = s.str();
          else if (f2 == 2 && wt2 == 0) v = int64_t(s.varint());
          else s.skip(wt2);
        }
        if (!fo) opsets.raw(",");
        fo = false;
        opsets.raw("{\"domain\":"); opsets.str(d); opsets.raw(",\"version\":"); opsets.i64(v); opsets.raw("}");
        break;
      }
      case 14: {
        if (wt != 2) throw ParseError("metadata_props wire type");
        std::string k, v;
        parse_kv(r.sub(), k, v);
        if (!fm) meta.raw(",");
        fm = false;
        meta.raw("["); meta.str(k); meta.raw(","); meta.str(v); meta.raw("]");
        break;
      }
      default: r.skip(wt);
    }
  }
  (void)has_ir;
  j.raw("{\"ir_version\":"); j.i64(ir_version);
  j.raw(",\"producer_name\":"); j.str(producer_name);
  j.raw(",\"producer_version\":"); j.str(producer_version);
  j.raw(",\"domain\":"); j.str(domain);
  j.raw(",\"model_version\":"); j.i64(model_version);
  j.raw(",\"doc_string\":"); j.str(doc);
  j.raw(",\"opset_import\":["); j.s += opsets.s;
  j.raw("],\"metadata_props\":["); j.s += meta.s;
  j.raw("],\"graph\":");
  j.s += has_graph ? graph_json : std::string("null");
  j.raw("}");
  out.json = std::move(j.s);
}

// ---------------------------------------------------------------- wire writer
struct Writer {
  std::string buf;
  void varint(uint64_t v) {
    while (v >= 0x80) { buf.push_back(char((v & 0x7f) | 0x80)); v >>= 7; }
    buf.push_back(char(v));
  }
  void tag(uint32_t field, uint32_t wt) { varint((uint64_t(field) << 3) | wt); }
  void f_varint(uint32_t field, uint64_t v) { tag(field, 0); varint(v); }
  void f_bytes(uint32_t field, const void* p, size_t n) {
    tag(field, 2); varint(n); buf.append(static_cast<const char*>(p), n);
  }
  void f_str(uint32_t field, const std::string& s) { f_bytes(field, s.data(), s.size()); }
  void f_msg(uint32_t field, const Writer& w) { f_bytes(field, w.buf.data(), w.buf.size()); }
  void f_f32(uint32_t field, float v) { tag(field, 5); buf.append(reinterpret_cast<const char*>(&v), 4); }
};

struct ModelBuilder {
  Writer graph;            // GraphProto under construction
  Writer model_head;       // ModelProto fields before the graph
  Writer model_tail;       // ModelProto fields after the graph
  Writer node;             // current NodeProto
  bool node_open = false;
  std::string result;
  void close_node() {
    if (node_open) { graph.f_msg(1, node); node = Writer(); node_open = false; }
  }
};

Writer make_tensor(const char* name, int32_t dtype, const int64_t* dims, int ndim,
                   const void* data, size_t nbytes) {
  Writer t;
  for (int i = 0; i < ndim; ++i) t.f_varint(1, uint64_t(dims[i]));
  t.f_varint(2, uint64_t(dtype));
  if (name && *name) t.f_str(8, name);
  t.f_bytes(9, data, nbytes);
  return t;
}

Writer make_value_info(const char* name, int32_t elem_type, int ndim, const int64_t* dims,
                       const char* const* dim_params) {
  Writer shape;
  for (int i = 0; i < ndim; ++i) {
    Writer d;
    if (dim_params && dim_params[i] && dim_params[i][0]) d.f_str(2, dim_params[i]);
    else d.f_varint(1, uint64_t(dims[i]));
    shape.f_msg(1, d);
  }
  Writer tt;
  tt.f_varint(1, uint64_t(elem_type));
  if (ndim >= 0) tt.f_msg(2, shape);
  Writer tp;
  tp.f_msg(1, tt);
  Writer vi;
  vi.f_str(1, name);
  vi.f_msg(2, tp);
  return vi;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ decode API
void* ronn_onnx_parse(const uint8_t* data, uint64_t n) {
  Parsed* p = new Parsed();
  try {
    if (data == nullptr || n == 0) throw ParseError("empty model buffer");
    parse_model(data, size_t(n), *p);
  } catch (const std::exception& e) {
    p->error = e.what();
    if (p->error.empty()) p->error = "parse error";
  }
  return p;
}
const char* ronn_onnx_error(void* h) {
  Parsed* p = static_cast<Parsed*>(h);
  return p->error.empty() ? nullptr : p->error.c_str();
}
const char* ronn_onnx_json(void* h, uint64_t* len) {
  Parsed* p = static_cast<Parsed*>(h);
  if (len) *len = p->json.size();
  return p->json.data();
}
uint64_t ronn_onnx_num_blobs(void* h) { return static_cast<Parsed*>(h)->blobs.size(); }
const uint8_t* ronn_onnx_blob(void* h, uint64_t i, uint64_t* len) {
  Parsed* p = static_cast<Parsed*>(h);
  if (i >= p->blobs.size()) { if (len) *len = 0; return nullptr; }
  if (len) *len = p->blobs[i].size();
  return p->blobs[i].data();
}
void ronn_onnx_free(void* h) { delete static_cast<Parsed*>(h); }
int ronn_onnx_elem_size(int32_t dt) { return elem_size(dt); }

// ------------------------------------------------------------------ encode API
void* ronn_onnxw_begin(int64_t ir_version, const char* producer_name, const char* producer_version,
                       const char* graph_name) {
  ModelBuilder* b = new ModelBuilder();
  b->model_head.f_varint(1, uint64_t(ir_version));
  if (producer_name && *producer_name) b->model_head.f_str(2, producer_name);
  if (producer_version && *producer_version) b->model_head.f_str(3, producer_version);
  if (graph_name && *graph_name) b->graph.f_str(2, graph_name);
  return b;
}
void ronn_onnxw_opset(void* h, const char* domain, int64_t version) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer o;
  if (domain && *domain) o.f_str(1, domain);
  o.f_varint(2, uint64_t(version));
  b->model_tail.f_msg(8, o);
}
void ronn_onnxw_metadata(void* h, const char* key, const char* value) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer kv;
  kv.f_str(1, key);
  kv.f_str(2, value);
  b->model_tail.f_msg(14, kv);
}
void ronn_onnxw_node(void* h, const char* name, const char* op_type, const char* domain,
                     const char* const* inputs, int n_in, const char* const* outputs, int n_out) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  b->close_node();
  b->node_open = true;
  for (int i = 0; i < n_in; ++i) b->node.f_str(1, inputs[i]);
  for (int i = 0; i < n_out; ++i) b->node.f_str(2, outputs[i]);
  if (name && *name) b->node.f_str(3, name);
  b->node.f_str(4, op_type);
  if (domain && *domain) b->node.f_str(7, domain);
}
void ronn_onnxw_attr_i(void* h, const char* name, int64_t v) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer a; a.f_str(1, name); a.f_varint(3, uint64_t(v)); a.f_varint(20, 2);
  b->node.f_msg(5, a);
}
void ronn_onnxw_attr_f(void* h, const char* name, float v) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer a; a.f_str(1, name); a.f_f32(2, v); a.f_varint(20, 1);
  b->node.f_msg(5, a);
}
void ronn_onnxw_attr_s(void* h, const char* name, const char* v, uint64_t n) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer a; a.f_str(1, name); a.f_bytes(4, v, size_t(n)); a.f_varint(20, 3);
  b->node.f_msg(5, a);
}
void ronn_onnxw_attr_ints(void* h, const char* name, const int64_t* v, int n) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer a; a.f_str(1, name);
  Writer packed;
  for (int i = 0; i < n; ++i) packed.varint(uint64_t(v[i]));
  a.f_bytes(8, packed.buf.data(), packed.buf.size());
  a.f_varint(20, 7);
  b->node.f_msg(5, a);
}
void ronn_onnxw_attr_floats(void* h, const char* name, const float* v, int n) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer a; a.f_str(1, name);
  a.f_bytes(7, v, size_t(n) * 4);
  a.f_varint(20, 6);
  b->node.f_msg(5, a);
}
void ronn_onnxw_attr_strings(void* h, const char* name, const char* const* v, int n) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer a; a.f_str(1, name);
  for (int i = 0; i < n; ++i) a.f_str(9, v[i]);
  a.f_varint(20, 8);
  b->node.f_msg(5, a);
}
void ronn_onnxw_attr_tensor(void* h, const char* name, int32_t dtype, const int64_t* dims, int ndim,
                            const void* data, uint64_t nbytes) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  Writer a; a.f_str(1, name);
  a.f_msg(5, make_tensor("", dtype, dims, ndim, data, size_t(nbytes)));
  a.f_varint(20, 4);
  b->node.f_msg(5, a);
}
void ronn_onnxw_initializer(void* h, const char* name, int32_t dtype, const int64_t* dims, int ndim,
                            const void* data, uint64_t nbytes) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  b->close_node();
  b->graph.f_msg(5, make_tensor(name, dtype, dims, ndim, data, size_t(nbytes)));
}
// kind: 0 = graph input, 1 = graph output, 2 = value_info
void ronn_onnxw_value(void* h, int kind, const char* name, int32_t elem_type, int ndim,
                      const int64_t* dims, const char* const* dim_params) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  b->close_node();
  uint32_t field = kind == 0 ? 11 : (kind == 1 ? 12 : 13);
  b->graph.f_msg(field, make_value_info(name, elem_type, ndim, dims, dim_params));
}
const char* ronn_onnxw_finish(void* h, uint64_t* len) {
  ModelBuilder* b = static_cast<ModelBuilder*>(h);
  b->close_node();
  Writer m;
  m.buf = b->model_head.buf;
  m.f_msg(7, b->graph);
  m.buf += b->model_tail.buf;
  b->result = std::move(m.buf);
  if (len) *len = b->result.size();
  return b->result.data();
}
void ronn_onnxw_free(void* h) { delete static_cast<ModelBuilder*>(h); }

}  // extern "C"
