// Recursive-descent reader for the textual MLIR that ryft-mlir prints.
//
// Accepted: `module { func.func @main(...) -> ... { ... } }` with the StableHLO
// ops listed in ir.h, each in its pretty form (the forms pinned by the printed
// -form tests under crates/ryft-mlir/src/dialects/stable_hlo/operations/) and
// in MLIR's generic form `"stablehlo.op"(%a) <{props}> ({regions}) : (T) -> T`
// (reference example: communication.rs:1759-1767).  Anything else is rejected
// with UNIMPLEMENTED naming the op; nothing is ever evaluated on the host.
#include <cmath>
#include <cstring>
#include <map>
#include <sstream>

#include "ir.h"

namespace b2x {

const char* dtype_name(DType t) {
  switch (t) {
    case DType::PRED: return "i1"; case DType::S8: return "i8"; case DType::S16: return "i16";
    case DType::S32: return "i32"; case DType::S64: return "i64"; case DType::U8: return "ui8";
    case DType::U16: return "ui16"; case DType::U32: return "ui32"; case DType::U64: return "ui64";
    case DType::F16: return "f16"; case DType::BF16: return "bf16"; case DType::F32: return "f32";
    case DType::F64: return "f64"; default: return "invalid";
  }
}

std::string TensorType::str() const {
  std::string s = "tensor<";
  for (auto d : dims) s += std::to_string(d) + "x";
  return s + dtype_name(dtype) + ">";
}

namespace {
struct OpInfo { const char* name; OpKind kind; int arity; bool elementwise; };
const OpInfo kOps[] = {
    {"negate", OpKind::NEGATE, 1, true}, {"abs", OpKind::ABS, 1, true}, {"tanh", OpKind::TANH, 1, true},
    {"exponential", OpKind::EXP, 1, true}, {"log", OpKind::LOG, 1, true}, {"sqrt", OpKind::SQRT, 1, true},
    {"rsqrt", OpKind::RSQRT, 1, true}, {"logistic", OpKind::LOGISTIC, 1, true}, {"not", OpKind::NOT, 1, true},
    {"convert", OpKind::CONVERT, 1, true}, {"sign", OpKind::SIGN, 1, true}, {"floor", OpKind::FLOOR, 1, true},
    {"ceil", OpKind::CEIL, 1, true}, {"exponential_minus_one", OpKind::EXPM1, 1, true},
    {"log_plus_one", OpKind::LOG1P, 1, true}, {"sine", OpKind::SINE, 1, true}, {"cosine", OpKind::COSINE, 1, true},
    {"add", OpKind::ADD, 2, true}, {"subtract", OpKind::SUBTRACT, 2, true}, {"multiply", OpKind::MULTIPLY, 2, true},
    {"divide", OpKind::DIVIDE, 2, true}, {"maximum", OpKind::MAXIMUM, 2, true}, {"minimum", OpKind::MINIMUM, 2, true},
    {"power", OpKind::POWER, 2, true}, {"and", OpKind::AND, 2, true}, {"or", OpKind::OR, 2, true},
    {"xor", OpKind::XOR, 2, true}, {"remainder", OpKind::REMAINDER, 2, true}, {"compare", OpKind::COMPARE, 2, true},
    {"select", OpKind::SELECT, 3, true}, {"clamp", OpKind::CLAMP, 3, true},
    {"constant", OpKind::CONSTANT, 0, true}, {"iota", OpKind::IOTA, 0, true},
    {"replica_id", OpKind::REPLICA_ID, 0, true}, {"partition_id", OpKind::PARTITION_ID, 0, true},
    {"broadcast_in_dim", OpKind::BROADCAST_IN_DIM, 1, false}, {"transpose", OpKind::TRANSPOSE, 1, false},
    {"reshape", OpKind::RESHAPE, 1, false}, {"dot_general", OpKind::DOT_GENERAL, 2, false},
    {"reduce", OpKind::REDUCE, -1, false}, {"all_reduce", OpKind::ALL_REDUCE, -1, false},
    {"all_gather", OpKind::ALL_GATHER, -1, false}, {"return", OpKind::RETURN, -1, false},
};
const OpInfo* find_op(const std::string& short_name) {
  for (auto& o : kOps) if (short_name == o.name) return &o;
  return nullptr;
}
const OpInfo& info_of(OpKind k) {
  for (auto& o : kOps) if (o.kind == k) return o;
  return kOps[0];
}
}  // namespace

const char* op_name(OpKind k) {
  static std::map<OpKind, std::string> names;
  if (names.empty()) for (auto& o : kOps) names[o.kind] = std::string("stablehlo.") + o.name;
  return names[k].c_str();
}
bool op_is_elementwise(OpKind k) { return info_of(k).elementwise; }

namespace {

// A generic attribute value: enough structure for the properties this subset reads.
struct Attr {
  enum Kind { NONE, INT, FLOAT, BOOL, STRING, ARRAY, DENSE, RAW } kind = NONE;
  int64_t i = 0;
  double f = 0;
  bool b = false;
  std::string s;            // STRING, or RAW text of an attribute this reader does not interpret
  std::vector<Attr> items;  // ARRAY
  // DENSE: flattened literals (text tokens) + whether the literal was a single (splat) scalar + the type
  std::vector<std::string> dense_tokens;
  bool dense_splat = false;
  bool dense_hex_blob = false;
  TensorType dense_type;
};

class Parser {
 public:
  explicit Parser(const std::string& text) : s_(text) {}

  std::unique_ptr<Module> parse() {
    mod_.reset(new Module());
    mod_->source = s_;
    skip_ws();
    bool in_module = false;
    if (try_word("module")) {
      in_module = true;
      skip_ws();
      if (peek() == '@') { next(); read_ident(); }
      if (try_word("attributes")) parse_attr_dict();
      expect('{');
    }
    bool seen_main = false;
    while (true) {
      skip_ws();
      if (eof()) break;
      if (peek() == '}') { if (in_module) { next(); } break; }
      if (try_word("func.func")) {
        if (seen_main) fail(kUnimplemented, "modules with more than one function are not supported");
        parse_func();
        seen_main = true;
      } else {
        fail(kInvalidArgument, "expected 'func.func' at module level");
      }
    }
    if (!seen_main) fail(kInvalidArgument, "the module contains no func.func");
    return std::move(mod_);
  }

 private:
  const std::string& s_;
  size_t p_ = 0;
  int line_ = 1;
  std::unique_ptr<Module> mod_;
  std::map<std::string, Value*> names_;  // SSA name (without '%') -> value

  [[noreturn]] void fail(int code, const std::string& msg) {
    throw CompileError(code, "MLIR parse error at line " + std::to_string(line_) + ": " + msg);
  }
  bool eof() const { return p_ >= s_.size(); }
  char peek(size_t off = 0) const { return p_ + off < s_.size() ? s_[p_ + off] : '\0'; }
  char next() { char c = s_[p_++]; if (c == '\n') line_++; return c; }
  void skip_ws() {
    while (!eof()) {
      char c = peek();
      if (c == ' ' || c == '\t' || c == '\r' || c == '\n') next();
      else if (c == '/' && peek(1) == '/') { while (!eof() && peek() != '\n') next(); }
      else break;
    }
  }
  void expect(char c) {
    skip_ws();
    if (peek() != c) fail(kInvalidArgument, std::string("expected '") + c + "' but found '" + (eof() ? std::string("<eof>") : std::string(1, peek())) + "'");
    next();
  }
  bool try_char(char c) { skip_ws(); if (peek() == c) { next(); return true; } return false; }
  static bool ident_char(char c) { return isalnum((unsigned char)c) || c == '_' || c == '.' || c == '$' || c == '-'; }
  bool try_word(const char* w) {
    skip_ws();
    size_t n = strlen(w);
    if (s_.compare(p_, n, w) == 0 && !ident_char(peek(n))) { p_ += n; return true; }
    return false;
  }
  std::string read_ident() {
    skip_ws();
    std::string r;
    if (peek() == '"') return read_string();
    while (!eof() && ident_char(peek())) r.push_back(next());
    if (r.empty()) fail(kInvalidArgument, "expected an identifier");
    return r;
  }
  std::string read_string() {
    expect('"');
    std::string r;
    while (!eof() && peek() != '"') {
      char c = next();
      if (c == '\\' && !eof()) {
        char d = next();
        if (d == 'n') r.push_back('\n');
        else if (d == 't') r.push_back('\t');
        else if (isxdigit((unsigned char)d) && isxdigit((unsigned char)peek())) {
          char e = next();
          r.push_back((char)std::stoi(std::string{d, e}, nullptr, 16));
        } else r.push_back(d);
      } else r.push_back(c);
    }
    expect('"');
    return r;
  }
  int64_t read_int() {
    skip_ws();
    std::string t;
    if (peek() == '-' || peek() == '+') t.push_back(next());
    while (isdigit((unsigned char)peek())) t.push_back(next());
    if (t.empty() || t == "-" || t == "+") fail(kInvalidArgument, "expected an integer");
    return std::stoll(t);
  }
  std::vector<int64_t> read_int_list() {  // [a, b, c]
    std::vector<int64_t> r;
    expect('[');
    if (try_char(']')) return r;
    do { r.push_back(read_int()); } while (try_char(','));
    expect(']');
    return r;
  }

  // ---- types -------------------------------------------------------------------------------
  DType parse_elem_type(const std::string& t) {
    static const std::map<std::string, DType> m = {
        {"i1", DType::PRED}, {"i8", DType::S8}, {"i16", DType::S16}, {"i32", DType::S32}, {"i64", DType::S64},
        {"si8", DType::S8}, {"si16", DType::S16}, {"si32", DType::S32}, {"si64", DType::S64},
        {"ui8", DType::U8}, {"ui16", DType::U16}, {"ui32", DType::U32}, {"ui64", DType::U64},
        {"f16", DType::F16}, {"bf16", DType::BF16}, {"f32", DType::F32}, {"f64", DType::F64}};
    auto it = m.find(t);
    if (it == m.end()) fail(kUnimplemented, "element type '" + t + "' is not supported by this executor");
    return it->second;
  }
  TensorType parse_type() {
    skip_ws();
    if (!try_word("tensor")) fail(kUnimplemented, "only ranked tensor types are supported, found '" + s_.substr(p_, 16) + "'");
    expect('<');
    TensorType t;
    while (true) {
      skip_ws();
      if (isdigit((unsigned char)peek())) {
        int64_t d = 0;
        while (isdigit((unsigned char)peek())) d = d * 10 + (next() - '0');
        if (peek() != 'x') fail(kInvalidArgument, "malformed tensor shape");
        next();
        t.dims.push_back(d);
      } else if (peek() == '?') {
        fail(kUnimplemented, "dynamic dimensions are not supported");
      } else break;
    }
    std::string e;
    while (!eof() && (isalnum((unsigned char)peek()))) e.push_back(next());
    if (e == "complex") fail(kUnimplemented, "complex element types are not supported");
    t.dtype = parse_elem_type(e);
    skip_ws();
    if (peek() == ',') {  // encoding attribute: skip to the closing '>'
      int depth = 1;
      while (!eof() && depth > 0) { char c = next(); if (c == '<') depth++; else if (c == '>') depth--; }
      return t;
    }
    expect('>');
    return t;
  }
  std::vector<TensorType> parse_type_list_parens() {  // (T, T)  or ()
    std::vector<TensorType> r;
    expect('(');
    if (try_char(')')) return r;
    do { r.push_back(parse_type()); } while (try_char(','));
    expect(')');
    return r;
  }
  // "(T, T) -> T" | "(T) -> (T, T)"
  void parse_function_type(std::vector<TensorType>* ins, std::vector<TensorType>* outs) {
    *ins = parse_type_list_parens();
    skip_ws();
    if (!(peek() == '-' && peek(1) == '>')) fail(kInvalidArgument, "expected '->' in function type");
    p_ += 2;
    skip_ws();
    if (peek() == '(') *outs = parse_type_list_parens();
    else outs->assign(1, parse_type());
  }

  // ---- attributes --------------------------------------------------------------------------
  // Skips a balanced run starting at an opening bracket character.
  std::string skip_balanced() {
    size_t start = p_;
    int depth = 0;
    while (!eof()) {
      char c = peek();
      if (c == '"') { read_string(); continue; }
      if (c == '<' || c == '[' || c == '(' || c == '{') depth++;
      else if (c == '>' || c == ']' || c == ')' || c == '}') { depth--; if (depth == 0) { next(); break; } }
      else if (c == '-' && peek(1) == '>') { next(); }
      next();
    }
    return s_.substr(start, p_ - start);
  }

  void collect_dense_tokens(Attr* a) {
    skip_ws();
    if (peek() == '[') {
      next();
      if (try_char(']')) return;
      do { collect_dense_tokens(a); } while (try_char(','));
      expect(']');
    } else {
      std::string t;
      while (!eof() && (isalnum((unsigned char)peek()) || peek() == '.' || peek() == '-' || peek() == '+')) t.push_back(next());
      if (t.empty()) fail(kInvalidArgument, "malformed dense literal");
      a->dense_tokens.push_back(t);
    }
  }

  Attr parse_attr_value() {
    skip_ws();
    Attr a;
    char c = peek();
    if (c == '"') { a.kind = Attr::STRING; a.s = read_string(); maybe_skip_type_suffix(); return a; }
    if (c == '[') {
      a.kind = Attr::ARRAY;
      next();
      if (try_char(']')) return a;
      do { a.items.push_back(parse_attr_value()); } while (try_char(','));
      expect(']');
      return a;
    }
    if (c == '#' || c == '{' || c == '<' || c == '(' || c == '@') {
      a.kind = Attr::RAW;
      size_t start = p_;
      if (c == '#' || c == '@') { next(); while (!eof() && (ident_char(peek()))) next(); skip_ws_inline(); }
      if (peek() == '<' || peek() == '{' || peek() == '(') skip_balanced();
      a.s = s_.substr(start, p_ - start);
      return a;
    }
    if (try_word("dense")) {
      a.kind = Attr::DENSE;
      expect('<');
      skip_ws();
      if (peek() == '"') { a.dense_hex_blob = true; a.dense_tokens.push_back(read_string()); }
      else if (peek() == '>') { /* empty */ }
      else { a.dense_splat = (peek() != '['); collect_dense_tokens(&a); }
      expect('>');
      expect(':');
      a.dense_type = parse_type();
      return a;
    }
    if (try_word("array")) {  // array<i64: 1, 2>
      a.kind = Attr::ARRAY;
      expect('<');
      read_ident();
      if (try_char(':')) {
        do { Attr e; e.kind = Attr::INT; e.i = read_int(); a.items.push_back(e); } while (try_char(','));
      }
      expect('>');
      return a;
    }
    if (try_word("true")) { a.kind = Attr::BOOL; a.b = true; maybe_skip_type_suffix(); return a; }
    if (try_word("false")) { a.kind = Attr::BOOL; a.b = false; maybe_skip_type_suffix(); return a; }
    if (try_word("unit")) { a.kind = Attr::BOOL; a.b = true; return a; }
    if (isdigit((unsigned char)c) || c == '-' || c == '+') {
      std::string t;
      while (!eof() && (isalnum((unsigned char)peek()) || peek() == '.' || peek() == '-' || peek() == '+')) t.push_back(next());
      if (t.find_first_of(".eE") != std::string::npos && t.compare(0, 2, "0x") != 0) { a.kind = Attr::FLOAT; a.f = std::stod(t); }
      else { a.kind = Attr::INT; a.i = std::stoll(t, nullptr, 0); }
      maybe_skip_type_suffix();
      return a;
    }
    // bare identifier / type-like attribute (e.g. `f32`, `tensor<...>`): keep raw
    a.kind = Attr::RAW;
    size_t start = p_;
    while (!eof() && ident_char(peek())) next();
    if (peek() == '<') skip_balanced();
    a.s = s_.substr(start, p_ - start);
    if (a.s.empty()) fail(kInvalidArgument, "malformed attribute value");
    return a;
  }
  void skip_ws_inline() { while (peek() == ' ' || peek() == '\t') next(); }
  void maybe_skip_type_suffix() {  // `: i64`, `: tensor<...>`
    skip_ws();
    if (peek() == ':' ) {
      size_t save = p_; int save_line = line_;
      next(); skip_ws();
      if (isalpha((unsigned char)peek())) {
        while (!eof() && ident_char(peek())) next();
        if (peek() == '<') skip_balanced();
      } else { p_ = save; line_ = save_line; }
    }
  }
  // { name = value, name, ... }  or  <{ ... }>
  std::map<std::string, Attr> parse_attr_dict() {
    std::map<std::string, Attr> d;
    expect('{');
    if (try_char('}')) return d;
    do {
      std::string k = read_ident();
      Attr v;
      if (try_char('=')) v = parse_attr_value();
      else { v.kind = Attr::BOOL; v.b = true; }  // unit attribute
      d[k] = v;
    } while (try_char(','));
    expect('}');
    return d;
  }

  // ---- SSA values --------------------------------------------------------------------------
  std::string read_ssa_name() {  // %name or %name#k
    skip_ws();
    if (peek() != '%') fail(kInvalidArgument, "expected an SSA value");
    next();
    std::string r;
    while (!eof() && (ident_char(peek()) || peek() == '#')) r.push_back(next());
    return r;
  }
  Value* lookup(const std::string& n) {
    auto it = names_.find(n);
    if (it == names_.end()) {
      // `%0#1` form when the definition registered `%0` with several results is registered as "0#1" already.
      fail(kInvalidArgument, "use of undefined value %" + n);
    }
    return it->second;
  }
  Value* read_operand() { return lookup(read_ssa_name()); }

  // ---- constants ---------------------------------------------------------------------------
  static void put_bytes(std::vector<uint8_t>* out, const void* p, size_t n) {
    const uint8_t* b = (const uint8_t*)p;
    out->insert(out->end(), b, b + n);
  }
  static uint16_t f32_to_bf16_rne(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1);
    return (uint16_t)(u >> 16);
  }
  static uint16_t f32_to_f16_rne(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    uint32_t man = x & 0x7fffffu;
    if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0) {
      if (exp < -10) return (uint16_t)sign;
      man |= 0x800000u;
      uint32_t shift = (uint32_t)(14 - exp);
      uint32_t r = man >> shift;
      uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
      if (rem > half || (rem == half && (r & 1))) r++;
      return (uint16_t)(sign | r);
    }
    uint32_t r = (uint32_t)(exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r++;
    return (uint16_t)(sign | r);
  }
  void encode_literal(const std::string& tok, DType dt, std::vector<uint8_t>* out) {
    bool is_hex = tok.size() > 2 && tok[0] == '0' && (tok[1] == 'x' || tok[1] == 'X');
    if (dtype_is_float(dt)) {
      if (is_hex) {  // bit pattern of the element type (crates/ryft-mlir/src/dialects/builtin/attributes/float.rs:12-24)
        uint64_t bits = std::stoull(tok, nullptr, 16);
        put_bytes(out, &bits, dtype_size(dt));
        return;
      }
      double v;
      if (tok == "true") v = 1; else if (tok == "false") v = 0; else {
        try { v = std::stod(tok); } catch (...) { fail(kInvalidArgument, "malformed float literal '" + tok + "'"); }
      }
      if (dt == DType::F64) put_bytes(out, &v, 8);
      else if (dt == DType::F32) { float f = (float)v; put_bytes(out, &f, 4); }
      else if (dt == DType::BF16) { uint16_t h = f32_to_bf16_rne((float)v); put_bytes(out, &h, 2); }
      else { uint16_t h = f32_to_f16_rne((float)v); put_bytes(out, &h, 2); }
      return;
    }
    int64_t v;
    if (tok == "true") v = 1; else if (tok == "false") v = 0; else {
      try { v = (int64_t)std::stoull(tok[0] == '-' ? tok.substr(1) : tok, nullptr, 0); if (tok[0] == '-') v = -v; }
      catch (...) { fail(kInvalidArgument, "malformed integer literal '" + tok + "'"); }
    }
    if (dt == DType::PRED) { uint8_t b = v != 0; put_bytes(out, &b, 1); }
    else put_bytes(out, &v, dtype_size(dt));
  }
  void fill_constant(Op* op, const Attr& a) {
    if (a.kind != Attr::DENSE) fail(kUnimplemented, "only dense<...> constants are supported");
    const TensorType& t = a.dense_type;
    int es = dtype_size(t.dtype);
    if (a.dense_hex_blob) {
      const std::string& h = a.dense_tokens[0];
      if (h.size() < 2 || h[0] != '0' || h[1] != 'x') fail(kInvalidArgument, "malformed hex constant blob");
      for (size_t i = 2; i + 1 < h.size(); i += 2) op->const_data.push_back((uint8_t)std::stoi(h.substr(i, 2), nullptr, 16));
      if ((int64_t)op->const_data.size() == es) op->splat = true;
      else if ((int64_t)op->const_data.size() != t.byte_size()) fail(kInvalidArgument, "hex constant blob size does not match its type");
      return;
    }
    for (auto& tok : a.dense_tokens) encode_literal(tok, t.dtype, &op->const_data);
    int64_t n = (int64_t)a.dense_tokens.size();
    if (a.dense_splat || (n == 1 && t.num_elements() != 1)) op->splat = true;
    else if (n != t.num_elements()) fail(kInvalidArgument, "dense literal has " + std::to_string(n) + " elements but its type " + t.str() + " needs " + std::to_string(t.num_elements()));
    if (t.num_elements() == 1) op->splat = true;
  }

  // ---- function ----------------------------------------------------------------------------
  void note_arg_attrs(const std::map<std::string, Attr>& d) {
    for (auto& kv : d)
      if (kv.first.compare(0, 4, "sdy.") == 0 || kv.first == "mhlo.sharding") mod_->has_sharding_attrs = true;
  }
  void parse_func() {
    if (try_word("public") || try_word("private")) {}
    skip_ws();
    expect('@');
    mod_->name = read_ident();
    expect('(');
    if (!try_char(')')) {
      do {
        std::string n = read_ssa_name();
        expect(':');
        TensorType t = parse_type();
        skip_ws();
        if (peek() == '{') note_arg_attrs(parse_attr_dict());
        if (try_word("loc")) skip_balanced();
        Value* v = mod_->new_value(t);
        v->arg_index = (int)mod_->args.size();
        v->name = n;
        mod_->args.push_back(v);
        names_[n] = v;
      } while (try_char(','));
      expect(')');
    }
    skip_ws();
    if (peek() == '-' && peek(1) == '>') {
      p_ += 2;
      skip_ws();
      if (peek() == '(') {
        next();
        if (!try_char(')')) {
          do { parse_type(); skip_ws(); if (peek() == '{') note_arg_attrs(parse_attr_dict()); } while (try_char(','));
          expect(')');
        }
      } else {
        parse_type();
        skip_ws();
      }
    }
    if (try_word("attributes")) note_arg_attrs(parse_attr_dict());
    expect('{');
    while (true) {
      skip_ws();
      if (peek() == '}') { next(); break; }
      if (eof()) fail(kInvalidArgument, "unterminated function body");
      parse_op_statement();
    }
    if (mod_->ops.empty() || mod_->ops.back()->kind != OpKind::RETURN) fail(kInvalidArgument, "function body does not end in a return");
  }

  Op* new_op(OpKind k) {
    mod_->ops.emplace_back(new Op());
    Op* op = mod_->ops.back().get();
    op->kind = k;
    op->line = line_;
    return op;
  }
  void add_result(Op* op, const TensorType& t) {
    Value* v = mod_->new_value(t);
    v->def = op;
    v->result_index = (int)op->results.size();
    op->results.push_back(v);
  }
  void add_operand(Op* op, Value* v) { op->operands.push_back(v); v->users.push_back(op); }

  void bind_results(Op* op, const std::vector<std::string>& lhs, int declared_count) {
    if (op->kind == OpKind::RETURN) return;
    if (lhs.empty()) return;
    if (lhs.size() == 1 && declared_count > 1) {
      if ((int)op->results.size() != declared_count) fail(kInvalidArgument, "result count mismatch");
      for (int i = 0; i < declared_count; i++) {
        names_[lhs[0] + "#" + std::to_string(i)] = op->results[i];
        op->results[i]->name = lhs[0] + "#" + std::to_string(i);
      }
      return;
    }
    if (lhs.size() != op->results.size()) fail(kInvalidArgument, std::string(op_name(op->kind)) + " defines " + std::to_string(op->results.size()) + " results but " + std::to_string(lhs.size()) + " names are bound");
    for (size_t i = 0; i < lhs.size(); i++) { names_[lhs[i]] = op->results[i]; op->results[i]->name = lhs[i]; }
  }

  void parse_op_statement() {
    std::vector<std::string> lhs;
    int declared = 1;
    skip_ws();
    if (peek() == '%') {
      do {
        std::string n = read_ssa_name();
        skip_ws();
        if (peek() == ':') { next(); declared = (int)read_int(); }
        lhs.push_back(n);
      } while (try_char(','));
      expect('=');
    }
    skip_ws();
    Op* op;
    if (peek() == '"') op = parse_generic_op();
    else op = parse_pretty_op();
    skip_ws();
    if (try_word("loc")) skip_balanced();
    bind_results(op, lhs, declared);
  }

  static Monoid monoid_of(OpKind k, bool* ok) {
    *ok = true;
    switch (k) {
      case OpKind::ADD: return Monoid::ADD; case OpKind::MULTIPLY: return Monoid::MUL;
      case OpKind::MAXIMUM: return Monoid::MAX; case OpKind::MINIMUM: return Monoid::MIN;
      case OpKind::AND: return Monoid::AND; case OpKind::OR: return Monoid::OR; case OpKind::XOR: return Monoid::XOR;
      default: *ok = false; return Monoid::ADD;
    }
  }

  // Reads a reducer region `{ ^bb0(%a: T, %b: T): %r = stablehlo.<op> %a, %b : T  stablehlo.return %r : T }` (braces
  // included) and returns its monoid.  Only single-op bodies that combine the two block arguments are executable.
  Monoid parse_reducer_region() {
    expect('{');
    std::map<std::string, Value*> saved = names_;
    skip_ws();
    std::vector<std::string> bargs;
    if (peek() == '^') {
      next(); read_ident();
      expect('(');
      do { bargs.push_back(read_ssa_name()); expect(':'); parse_type(); if (try_word("loc")) skip_balanced(); } while (try_char(','));
      expect(')');
      expect(':');
    }
    Monoid m = Monoid::ADD;
    bool found = false;
    while (true) {
      skip_ws();
      if (peek() == '}') { next(); break; }
      if (eof()) fail(kInvalidArgument, "unterminated region");
      // statement: [%r =] opname ...
      std::string res;
      if (peek() == '%') { res = read_ssa_name(); expect('='); }
      skip_ws();
      std::string name = peek() == '"' ? read_string() : read_ident();
      std::string shortn = name.compare(0, 10, "stablehlo.") == 0 ? name.substr(10) : name;
      if (shortn == "return" || name == "func.return") {
        // skip the rest of the line
        while (!eof() && peek() != '\n' && peek() != '}') next();
        continue;
      }
      const OpInfo* oi = find_op(shortn);
      bool ok = false;
      if (oi) m = monoid_of(oi->kind, &ok);
      if (!ok || found) fail(kUnimplemented, "reduction bodies other than a single add/multiply/maximum/minimum/and/or/xor are not supported (found '" + name + "')");
      found = true;
      while (!eof() && peek() != '\n') next();
    }
    if (!found) fail(kUnimplemented, "empty reduction body");
    names_ = saved;
    return m;
  }
  // reducer(%a: T, %b: T) { ... }  (pretty non-compact reduce form)
  Monoid parse_reducer_clause() {
    expect('(');
    int depth = 1;
    while (!eof() && depth > 0) { char c = next(); if (c == '(') depth++; else if (c == ')') depth--; }
    return parse_reducer_region();
  }

  static std::vector<int64_t> attr_ints(const Attr& a) {
    std::vector<int64_t> r;
    if (a.kind == Attr::ARRAY) for (auto& e : a.items) r.push_back(e.i);
    else if (a.kind == Attr::DENSE) for (auto& t : a.dense_tokens) r.push_back(std::stoll(t));
    else if (a.kind == Attr::INT) r.push_back(a.i);
    return r;
  }
  // #stablehlo.dot<lhs_batching_dimensions = [0], rhs_batching_dimensions = [0], lhs_contracting_dimensions = [2], ...>
  void parse_dot_dims_attr(const std::string& raw, Op* op) {
    auto grab = [&](const char* key, std::vector<int64_t>* out) {
      size_t k = raw.find(key);
      if (k == std::string::npos) return;
      size_t lb = raw.find('[', k), rb = raw.find(']', k);
      if (lb == std::string::npos || rb == std::string::npos) return;
      std::stringstream ss(raw.substr(lb + 1, rb - lb - 1));
      std::string tok;
      while (std::getline(ss, tok, ',')) if (tok.find_first_of("0123456789") != std::string::npos) out->push_back(std::stoll(tok));
    };
    grab("lhs_batching_dimensions", &op->lhs_batch);
    grab("rhs_batching_dimensions", &op->rhs_batch);
    grab("lhs_contracting_dimensions", &op->lhs_contract);
    grab("rhs_contracting_dimensions", &op->rhs_contract);
  }
  void apply_replica_groups(const Attr& a, Op* op) {
    if (a.kind != Attr::DENSE) fail(kInvalidArgument, "replica_groups must be a dense attribute");
    const TensorType& t = a.dense_type;
    int64_t rows = t.rank() == 2 ? t.dims[0] : 1, cols = t.rank() == 2 ? t.dims[1] : t.num_elements();
    std::vector<int64_t> flat;
    for (auto& tok : a.dense_tokens) flat.push_back(std::stoll(tok));
    if (a.dense_splat && !flat.empty()) flat.assign((size_t)(rows * cols), flat[0]);
    if ((int64_t)flat.size() != rows * cols) fail(kInvalidArgument, "replica_groups literal does not match its type");
    for (int64_t r = 0; r < rows; r++) {
      std::vector<int64_t> g;
      for (int64_t c = 0; c < cols; c++) if (flat[r * cols + c] >= 0) g.push_back(flat[r * cols + c]);  // -1 pads
      op->replica_groups.push_back(g);
    }
  }
  static CmpDir cmp_dir_of(const std::string& s, bool* ok) {
    *ok = true;
    if (s.find("EQ") != std::string::npos) return CmpDir::EQ;
    if (s.find("NE") != std::string::npos) return CmpDir::NE;
    if (s.find("GE") != std::string::npos) return CmpDir::GE;
    if (s.find("GT") != std::string::npos) return CmpDir::GT;
    if (s.find("LE") != std::string::npos) return CmpDir::LE;
    if (s.find("LT") != std::string::npos) return CmpDir::LT;
    *ok = false; return CmpDir::EQ;
  }
  static CmpType cmp_type_of(const std::string& s) {
    if (s.find("TOTALORDER") != std::string::npos) return CmpType::TOTALORDER;
    if (s.find("UNSIGNED") != std::string::npos) return CmpType::UNSIGNED;
    if (s.find("SIGNED") != std::string::npos) return CmpType::SIGNED;
    if (s.find("FLOAT") != std::string::npos) return CmpType::FLOAT;
    return CmpType::DEFAULT;
  }

  void apply_props(Op* op, const std::map<std::string, Attr>& d) {
    for (auto& kv : d) {
      const std::string& k = kv.first;
      const Attr& a = kv.second;
      if (k == "value" && op->kind == OpKind::CONSTANT) fill_constant(op, a);
      else if (k == "iota_dimension") op->iota_dim = a.i;
      else if (k == "broadcast_dimensions" || k == "permutation" || k == "dimensions") op->dims = attr_ints(a);
      else if (k == "comparison_direction") { bool ok; op->cmp_dir = cmp_dir_of(a.s, &ok); if (!ok) fail(kInvalidArgument, "bad comparison_direction"); }
      else if (k == "compare_type") op->cmp_type = cmp_type_of(a.s);
      else if (k == "dot_dimension_numbers") parse_dot_dims_attr(a.s, op);
      else if (k == "replica_groups") apply_replica_groups(a, op);
      else if (k == "channel_handle") op->has_channel = true;
      else if (k == "use_global_device_ids") op->use_global_device_ids = true;
      else if (k == "all_gather_dim") op->iota_dim = a.i;
      // precision_config, algorithm, result_accuracy, frontend attributes: accepted and ignored
    }
  }

  Op* parse_generic_op() {
    std::string name = read_string();
    std::string shortn;
    if (name.compare(0, 10, "stablehlo.") == 0) shortn = name.substr(10);
    else if (name == "func.return") shortn = "return";
    else fail(kUnimplemented, "operation '" + name + "' is not supported by this executor");
    const OpInfo* oi = find_op(shortn);
    if (!oi) fail(kUnimplemented, "operation '" + name + "' is not supported by this executor");
    Op* op = new_op(oi->kind);
    expect('(');
    if (!try_char(')')) {
      do { add_operand(op, read_operand()); } while (try_char(','));
      expect(')');
    }
    skip_ws();
    std::map<std::string, Attr> props;
    if (peek() == '<' && peek(1) == '{') { next(); props = parse_attr_dict(); expect('>'); }
    skip_ws();
    bool has_region = false;
    if (peek() == '(' ) {  // region list
      next();
      skip_ws();
      if (peek() == '{') { op->monoid = parse_reducer_region(); has_region = true; }
      expect(')');
    }
    skip_ws();
    if (peek() == '{') { auto more = parse_attr_dict(); for (auto& kv : more) props[kv.first] = kv.second; }
    apply_props(op, props);
    expect(':');
    std::vector<TensorType> ins, outs;
    parse_function_type(&ins, &outs);
    if (ins.size() != op->operands.size()) fail(kInvalidArgument, name + ": operand count does not match its function type");
    for (size_t i = 0; i < ins.size(); i++)
      if (ins[i] != op->operands[i]->type) fail(kInvalidArgument, name + ": operand " + std::to_string(i) + " has type " + op->operands[i]->type.str() + " but the op states " + ins[i].str());
    if (op->kind != OpKind::RETURN) for (auto& t : outs) add_result(op, t);
    if ((op->kind == OpKind::REDUCE || op->kind == OpKind::ALL_REDUCE) && !has_region) fail(kInvalidArgument, name + " needs a reduction body");
    finish_return(op);
    return op;
  }

  void finish_return(Op* op) {
    if (op->kind == OpKind::RETURN) mod_->outputs = op->operands;
  }

  // `: T` (all operands and the result share T) or `: (T, ...) -> T`
  void parse_same_or_function_type(Op* op) {
    expect(':');
    skip_ws();
    if (peek() == '(') {
      std::vector<TensorType> ins, outs;
      parse_function_type(&ins, &outs);
      if (ins.size() != op->operands.size()) fail(kInvalidArgument, std::string(op_name(op->kind)) + ": operand count does not match its type signature");
      for (size_t i = 0; i < ins.size(); i++)
        if (ins[i] != op->operands[i]->type) fail(kInvalidArgument, std::string(op_name(op->kind)) + ": operand " + std::to_string(i) + " has type " + op->operands[i]->type.str() + " but the op states " + ins[i].str());
      for (auto& t : outs) add_result(op, t);
    } else {
      TensorType t = parse_type();
      add_result(op, t);
    }
  }

  Op* parse_pretty_op() {
    std::string name = read_ident();
    std::string shortn;
    if (name == "return" || name == "func.return") shortn = "return";
    else if (name.compare(0, 10, "stablehlo.") == 0) shortn = name.substr(10);
    else fail(kUnimplemented, "operation '" + name + "' is not supported by this executor");
    const OpInfo* oi = find_op(shortn);
    if (!oi) fail(kUnimplemented, "operation '" + name + "' is not supported by this executor");
    Op* op = new_op(oi->kind);
    switch (oi->kind) {
      case OpKind::RETURN: {
        skip_ws();
        if (peek() == '%') {
          do { add_operand(op, read_operand()); } while (try_char(','));
          expect(':');
          size_t i = 0;
          do {
            TensorType t = parse_type();
            if (i < op->operands.size() && t != op->operands[i]->type) fail(kInvalidArgument, "return operand " + std::to_string(i) + " has type " + op->operands[i]->type.str() + " but is returned as " + t.str());
            i++;
          } while (try_char(','));
        }
        finish_return(op);
        break;
      }
      case OpKind::CONSTANT: {
        skip_ws();
        if (peek() == '{') parse_attr_dict();
        Attr a = parse_attr_value();
        fill_constant(op, a);
        add_result(op, a.dense_type);
        break;
      }
      case OpKind::IOTA: {
        if (!try_word("dim")) fail(kInvalidArgument, "expected 'dim' in stablehlo.iota");
        expect('=');
        op->iota_dim = read_int();
        expect(':');
        add_result(op, parse_type());
        break;
      }
      case OpKind::REPLICA_ID: case OpKind::PARTITION_ID: {
        expect(':');
        add_result(op, parse_type());
        break;
      }
      case OpKind::COMPARE: {
        bool ok;
        op->cmp_dir = cmp_dir_of(read_ident(), &ok);
        if (!ok) fail(kInvalidArgument, "bad comparison direction");
        expect(',');
        add_operand(op, read_operand());
        expect(',');
        add_operand(op, read_operand());
        if (try_char(',')) op->cmp_type = cmp_type_of(read_ident());
        parse_same_or_function_type(op);
        break;
      }
      case OpKind::SELECT: {
        add_operand(op, read_operand()); expect(',');
        add_operand(op, read_operand()); expect(',');
        add_operand(op, read_operand());
        expect(':');
        skip_ws();
        if (peek() == '(') {
          std::vector<TensorType> ins, outs;
          parse_function_type(&ins, &outs);
          for (auto& t : outs) add_result(op, t);
        } else {
          TensorType p = parse_type();
          if (try_char(',')) { TensorType r = parse_type(); add_result(op, r); }
          else add_result(op, op->operands[1]->type), (void)p;
        }
        break;
      }
      case OpKind::BROADCAST_IN_DIM: case OpKind::TRANSPOSE: {
        add_operand(op, read_operand());
        expect(',');
        if (!try_word("dims")) fail(kInvalidArgument, "expected 'dims'");
        expect('=');
        op->dims = read_int_list();
        parse_same_or_function_type(op);
        break;
      }
      case OpKind::RESHAPE: {
        add_operand(op, read_operand());
        parse_same_or_function_type(op);
        break;
      }
      case OpKind::DOT_GENERAL: {
        add_operand(op, read_operand()); expect(',');
        add_operand(op, read_operand());
        while (try_char(',')) {
          std::string key = read_ident();
          expect('=');
          if (key == "batching_dims") { op->lhs_batch = read_int_list(); if (!try_word("x")) fail(kInvalidArgument, "expected 'x'"); op->rhs_batch = read_int_list(); }
          else if (key == "contracting_dims") { op->lhs_contract = read_int_list(); if (!try_word("x")) fail(kInvalidArgument, "expected 'x'"); op->rhs_contract = read_int_list(); }
          else { parse_attr_value(); }  // precision = [DEFAULT, DEFAULT], algorithm = <...>
        }
        skip_ws();
        if (peek() == '{') parse_attr_dict();
        parse_same_or_function_type(op);
        break;
      }
      case OpKind::REDUCE: {
        // stablehlo.reduce(%x init: %i) [applies stablehlo.add] across dimensions = [1] : (T, T) -> T [reducer(...) {...}]
        expect('(');
        std::vector<Value*> ins, inits;
        do {
          ins.push_back(read_operand());
          if (!try_word("init")) fail(kInvalidArgument, "expected 'init:' in stablehlo.reduce");
          expect(':');
          inits.push_back(read_operand());
        } while (try_char(','));
        expect(')');
        for (auto v : ins) add_operand(op, v);
        for (auto v : inits) add_operand(op, v);
        bool have_body = false;
        if (try_word("applies")) {
          std::string body = read_ident();
          const OpInfo* bi = body.compare(0, 10, "stablehlo.") == 0 ? find_op(body.substr(10)) : nullptr;
          bool ok = false;
          if (bi) op->monoid = monoid_of(bi->kind, &ok);
          if (!ok) fail(kUnimplemented, "stablehlo.reduce body '" + body + "' is not supported");
          have_body = true;
        }
        if (!try_word("across")) fail(kInvalidArgument, "expected 'across dimensions' in stablehlo.reduce");
        if (!try_word("dimensions")) fail(kInvalidArgument, "expected 'dimensions'");
        expect('=');
        op->dims = read_int_list();
        parse_same_or_function_type(op);
        if (!have_body) {
          if (!try_word("reducer")) fail(kInvalidArgument, "stablehlo.reduce needs a body");
          op->monoid = parse_reducer_clause();
        }
        break;
      }
      case OpKind::ALL_REDUCE: case OpKind::ALL_GATHER:
        fail(kUnimplemented, std::string(op_name(oi->kind)) + " is only accepted in MLIR's generic form");
      default: {
        // unary / binary / ternary elementwise: operands, optional attr-dict, then the type
        skip_ws();
        if (peek() == '%') { do { add_operand(op, read_operand()); } while (try_char(',')); }
        skip_ws();
        if (peek() == '{') parse_attr_dict();
        if (oi->arity >= 0 && (int)op->operands.size() != oi->arity) fail(kInvalidArgument, name + " expects " + std::to_string(oi->arity) + " operands");
        parse_same_or_function_type(op);
        break;
      }
    }
    return op;
  }
};

}  // namespace

std::unique_ptr<Module> parse_module(const std::string& text) {
  if (text.size() >= 4 && (unsigned char)text[0] == 'M' && text[1] == 'L' && (unsigned char)text[2] == 0xEF && text[3] == 'R')
    throw CompileError(kUnimplemented,
                       "MLIR bytecode input is not supported by this executor yet; pass the module as text "
                       "(Operation::to_string()) through Program::Mlir instead");
  Parser p(text);
  auto m = p.parse();
  verify_module(*m);
  canonicalize(*m);
  verify_module(*m);
  return m;
}

}  // namespace b2x
