// StableHLO subset reader, dequant-chain matcher and launch plan.
//
// Stands where the reference has its MLIR-based parser and planner
// (src/pjrt_plugin/core/stablehlo_parser.mm:521-586,
//  src/pjrt_plugin/core/mps_executable.mm:7627-9008) for the one path this
// library covers.  It reads the textual form of a StableHLO module (what
// `jax.jit(f).lower(...).as_text()` prints; no MLIR libraries), builds an SSA
// table of the entry function, and — anchored on every stablehlo.dot_general,
// walking operands backwards the way the reference's tag-and-rewrite fusions do
// (mps_executable.mm:1214-1326) — recognises
//   P1  x @ (convert(W:i8) * broadcast(scale))            -> qmm_w8a32 / qmm_w8a16
//   P2  dot_general(A:i8, B:i8):i32 [-> convert * row * col] -> qmm_i8i8_i32
//   P3  x @ reshape((convert(unpack4(Wq)) - bcast(z)) * bcast(s)) -> qmm_w4a16_g128
// Each match becomes one kernel launch.  Ops that no match absorbs run as
// standalone GPU kernels (generic_ops.cu) if they belong to the small supported
// set (convert, multiply, subtract, add, and, shift_right_logical,
// broadcast_in_dim, reshape, transpose, slice, concatenate, constant, plain
// dot / dot_general), so that a dequantisation chain spelled in a way the
// matcher does not know still computes correctly, op by op; anything else is a
// compile error that names the op (the reference's convention,
// api/pjrt_client.cc:211-220).  Nothing ever runs on the CPU.  Dense constants
// (weights closed over by the jitted function) are lifted into extra arguments
// that the plan owns.  Every decision is recorded as a JSON line
// (`QMM_PLAN_JSON:`: "fused" with the kernel, "not_fused" with the op and, for a
// dot, the reason), like the reference's JAX_METALLIB_TRACE_PLAN output, so
// tests can assert that a chain was fused and fail on one that was not.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../common.cuh"
#include "../generic_ops.h"

namespace qmm {
namespace hlo {

struct TType {
  std::vector<int64_t> dims;
  std::string elem;
  bool ok = false;
  int64_t count() const {
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
};

struct Op {
  std::string result, name, body;  // body = operands + attributes, before the type signature
  std::vector<std::string> operands;
  std::vector<TType> in_types;
  TType out_type;
  int line = 0;
};

struct Module {
  std::vector<std::string> arg_names;
  std::vector<TType> arg_types;
  std::vector<Op> ops;
  std::vector<std::string> returns;
  std::map<std::string, int> def;   // SSA name -> op index
  std::map<std::string, int> argi;  // SSA name -> argument index
  int num_real_args = 0;            // arguments of @main; dense constants follow them as extra arguments
  std::vector<std::vector<uint8_t>> const_data;  // contents of the lifted constants, in argument order
  // Contiguous slices (and reshapes) of arguments are further extra arguments that alias their source:
  // (slot of the source, byte offset).  They follow the constants.  No data moves (the reference's
  // input-slice views, src/pjrt_plugin/core/mps_executable.mm:7509-7603).
  std::vector<std::pair<int, size_t>> views;
  std::set<int> view_ops;  // the ops these views stand for
  std::string name = "main";        // module symbol (jit_<function> in what jax prints)
  int num_replicas = 1, num_partitions = 1;  // mhlo.num_replicas / mhlo.num_partitions of the module
  std::string error;
};

static std::string trim(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\r\n");
  if (a == std::string::npos) return "";
  size_t b = s.find_last_not_of(" \t\r\n");
  return s.substr(a, b - a + 1);
}

// tensor<32x1024xf32>, tensor<f32>, tensor<2048x14336xui8>
static TType parse_type(const std::string& t0) {
  TType t;
  std::string s = trim(t0);
  if (s.compare(0, 7, "tensor<") != 0 || s.back() != '>') return t;
  s = s.substr(7, s.size() - 8);
  size_t pos = 0;
  while (true) {
    size_t x = s.find('x', pos);
    if (x == std::string::npos) break;
    std::string d = s.substr(pos, x - pos);
    if (d.empty() || d.find_first_not_of("0123456789") != std::string::npos) break;
    t.dims.push_back(atoll(d.c_str()));
    pos = x + 1;
  }
  t.elem = s.substr(pos);
  size_t comma = t.elem.find(',');
  if (comma != std::string::npos) t.elem = trim(t.elem.substr(0, comma));  // drop encodings
  t.ok = !t.elem.empty();
  return t;
}

// split at top-level commas
static std::vector<std::string> split_top(const std::string& s, char sep = ',') {
  std::vector<std::string> out;
  int depth = 0;
  std::string cur;
  for (char c : s) {
    if (c == '<' || c == '(' || c == '[' || c == '{') ++depth;
    if (c == '>' || c == ')' || c == ']' || c == '}') --depth;
    if (c == sep && depth == 0) {
      out.push_back(trim(cur));
      cur.clear();
    } else {
      cur += c;
    }
  }
  if (!trim(cur).empty()) out.push_back(trim(cur));
  return out;
}

// position of the last " : " at nesting depth 0 ("->" must not count as a closing '>')
static size_t last_top_colon(const std::string& s) {
  int depth = 0;
  size_t found = std::string::npos;
  for (size_t i = 0; i < s.size(); ++i) {
    char c = s[i];
    if (c == '"') {
      size_t e = s.find('"', i + 1);
      if (e == std::string::npos) break;
      i = e;
      continue;
    }
    if (c == '-' && i + 1 < s.size() && s[i + 1] == '>') {
      ++i;
      continue;
    }
    if (c == '<' || c == '(' || c == '[' || c == '{') ++depth;
    if (c == '>' || c == ')' || c == ']' || c == '}') --depth;
    if (c == ':' && depth == 0 && i > 0 && s[i - 1] == ' ' && i + 1 < s.size() && s[i + 1] == ' ')
      found = i;
  }
  return found;
}

static std::vector<int64_t> int_list_after(const std::string& s, const std::string& key, size_t from = 0,
                                           size_t* end = nullptr) {
  std::vector<int64_t> v;
  size_t p = s.find(key, from);
  if (p == std::string::npos) return v;
  size_t a = s.find('[', p);
  size_t b = s.find(']', a);
  if (a == std::string::npos || b == std::string::npos) return v;
  for (auto& tok : split_top(s.substr(a + 1, b - a - 1)))
    if (!tok.empty()) v.push_back(atoll(tok.c_str()));
  if (end) *end = b;
  return v;
}

static int dtype_of_elem_early(const std::string& e) {
  if (e == "f32") return QMM_F32;
  if (e == "f16") return QMM_F16;
  if (e == "bf16") return QMM_BF16;
  if (e == "i8" || e == "si8") return QMM_S8;
  if (e == "ui8") return QMM_U8;
  if (e == "i32" || e == "si32") return QMM_S32;
  if (e == "ui4") return QMM_U4;
  if (e == "ui32") return QMM_U32;
  return -1;
}

static void append_scalar(std::vector<uint8_t>& out, int dtype, double v) {
  auto put = [&](const void* p, size_t n) { out.insert(out.end(), (const uint8_t*)p, (const uint8_t*)p + n); };
  switch (dtype) {
    case QMM_F32: { float f = (float)v; put(&f, 4); break; }
    case QMM_BF16: {
      float f = (float)v;
      uint32_t u;
      memcpy(&u, &f, 4);
      uint32_t r = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;  // round to nearest even (finite values)
      if ((u & 0x7FFFFFFFu) > 0x7F800000u) r = ((u >> 16) & 0x8000u) | 0x7FC0u;
      uint16_t h = (uint16_t)r;
      put(&h, 2);
      break;
    }
    case QMM_S8: { int8_t x = (int8_t)(long long)v; put(&x, 1); break; }
    case QMM_U8: { uint8_t x = (uint8_t)(long long)v; put(&x, 1); break; }
    case QMM_S32: { int32_t x = (int32_t)(long long)v; put(&x, 4); break; }
    case QMM_U32: { uint32_t x = (uint32_t)(long long)v; put(&x, 4); break; }
    default: break;
  }
}

// The value of a stablehlo.constant: "dense<...>".  Returns 0 = splat (one value), 1 = dense
// (bytes filled, element count checked), -1 = not readable.
static int parse_dense(const std::string& body, const TType& t, std::vector<uint8_t>& bytes, std::string& err) {
  size_t a = body.find("dense<");
  if (a == std::string::npos) { err = "constant without a dense<...> value"; return -1; }
  size_t b = body.rfind('>');
  if (b == std::string::npos || b <= a + 6) { err = "malformed dense<...>"; return -1; }
  std::string val = trim(body.substr(a + 6, b - a - 6));
  if (val.empty()) { err = "empty dense<...>"; return -1; }
  const int dt = dtype_of_elem_early(t.elem);
  const int64_t count = t.count();
  if (val[0] == '"') {  // dense<"0x...">: the raw bytes of the tensor
    if (val.size() < 4 || val[1] != '0' || (val[2] != 'x' && val[2] != 'X') || val.back() != '"') {
      err = "unreadable hexadecimal constant";
      return -1;
    }
    const std::string hex = val.substr(3, val.size() - 4);
    if (hex.size() % 2) { err = "odd number of hexadecimal digits"; return -1; }
    for (size_t i = 0; i < hex.size(); i += 2) bytes.push_back((uint8_t)strtoul(hex.substr(i, 2).c_str(), nullptr, 16));
    const size_t bits = gen::dtype_bits(dt);
    if (dt < 0 || bytes.size() != (size_t)count * bits / 8) { err = "hexadecimal constant of the wrong size"; return -1; }
    return 1;
  }
  if (val[0] != '[') return 0;  // a splat: is_splat_const and the fill step read it from the body
  if (dt < 0 || dt == QMM_U4 || dt == QMM_F16) { err = "dense constant of element type " + t.elem + " is not supported"; return -1; }
  int64_t n = 0;
  for (size_t i = 0; i < val.size();) {
    const char c = val[i];
    if (c == '[' || c == ']' || c == ',' || c == ' ') { ++i; continue; }
    if (val.compare(i, 4, "true") == 0) { append_scalar(bytes, dt, 1); i += 4; ++n; continue; }
    if (val.compare(i, 5, "false") == 0) { append_scalar(bytes, dt, 0); i += 5; ++n; continue; }
    char* end = nullptr;
    const double v = strtod(val.c_str() + i, &end);
    if (end == val.c_str() + i) { err = "unreadable number in dense constant"; return -1; }
    append_scalar(bytes, dt, v);
    i = end - val.c_str();
    ++n;
  }
  if (n != count) { err = "dense constant has " + std::to_string(n) + " values, its type " + std::to_string(count); return -1; }
  return 1;
}

// ---------------------------------------------------------------------------
// Counted stablehlo.while loops are unrolled on the text, before the module is parsed, the way the
// reference unrolls them at parse time (src/pjrt_plugin/core/stablehlo_parser.mm:116-519: counted
// loops of a bounded trip count are replaced by their bodies, and dynamic_slice indices that depend
// only on the induction variable become static slices), so that a model written as a lax.scan over
// stacked per-layer weights reaches the matcher as straight-line code with one static slice per
// layer.  A loop is unrolled when every value its condition depends on folds to a constant: integer
// scalars are folded through constant, compare, add, subtract, multiply, select, convert, minimum,
// maximum, clamp, and, or.  The trip count is capped (kMaxUnrollTrips, like the reference's 16,
// raisable to 64).  Anything else about a while loop is an error naming the line.
// ---------------------------------------------------------------------------
struct SrcLine {
  std::string text;
  int line;
};
constexpr int kMaxUnrollTrips = 64;

static bool is_name_char(char c) { return isalnum((unsigned char)c) || c == '_' || c == '#'; }

// every %token of `s`, replaced through `sub` (longest names first is not needed: tokens are whole)
static std::string substitute(const std::string& s, const std::map<std::string, std::string>& sub) {
  std::string out;
  for (size_t i = 0; i < s.size();) {
    if (s[i] == '"') {  // string attributes are left alone
      size_t e = s.find('"', i + 1);
      e = e == std::string::npos ? s.size() : e + 1;
      out += s.substr(i, e - i);
      i = e;
      continue;
    }
    if (s[i] != '%') { out += s[i++]; continue; }
    size_t e = i + 1;
    while (e < s.size() && is_name_char(s[e])) ++e;
    const std::string tok = s.substr(i, e - i);
    auto it = sub.find(tok);
    out += it == sub.end() ? tok : it->second;
    i = e;
  }
  return out;
}

static bool scalar_int_type(const std::string& t) {
  return t == "tensor<i32>" || t == "tensor<i64>" || t == "tensor<i1>" || t == "tensor<ui32>" || t == "tensor<i8>" ||
         t == "tensor<ui8>" || t == "tensor<i16>";
}

struct Unroller {
  std::string err;
  int uid = 0;

  // Emits `in` into `out`, unrolling whiles; `known` = scalar integer values by SSA name; `sub` = renames.
  bool run(const std::vector<SrcLine>& in, std::vector<SrcLine>& out, std::map<std::string, long long>& known,
           std::map<std::string, std::string>& sub, int depth) {
    if (depth > 4) return fail(in.empty() ? 0 : in[0].line, "while loops nested too deeply");
    for (size_t i = 0; i < in.size(); ++i) {
      std::string l = substitute(trim(in[i].text), sub);
      size_t loc = l.find(" loc(");
      if (loc != std::string::npos) l = trim(l.substr(0, loc));
      const int ln = in[i].line;
      if (l.find("stablehlo.while") == std::string::npos || l.empty() || l[0] != '%') {
        if (!fold_or_emit(l, ln, out, known)) return false;
        continue;
      }
      // ---- %r:n = stablehlo.while(%iterArg = %init, ...) : types
      size_t eq = l.find(" = ");
      std::string res = trim(l.substr(0, eq));
      int nres = 1;
      size_t colon = res.find(':');
      if (colon != std::string::npos) {
        nres = atoi(res.c_str() + colon + 1);
        res = res.substr(0, colon);
      }
      size_t a = l.find('(', eq), b = l.find(')', a);
      if (a == std::string::npos || b == std::string::npos) return fail(ln, "malformed stablehlo.while");
      std::vector<std::string> iter_names, init;
      for (auto& pr : split_top(l.substr(a + 1, b - a - 1))) {
        size_t e2 = pr.find('=');
        if (e2 == std::string::npos) return fail(ln, "malformed stablehlo.while operand list");
        iter_names.push_back(trim(pr.substr(0, e2)));
        init.push_back(trim(pr.substr(e2 + 1)));
      }
      if ((int)iter_names.size() != nres) return fail(ln, "stablehlo.while: result count does not match its operands");
      size_t tc = l.find(" : ", b);
      std::vector<std::string> types = tc == std::string::npos ? std::vector<std::string>() : split_top(l.substr(tc + 3));
      if ((int)types.size() != nres) return fail(ln, "stablehlo.while: one type per loop-carried value expected");
      // ---- regions
      std::vector<SrcLine> cond, body;
      size_t j = i + 1;
      auto is_open = [&](const std::string& t, const char* what) { return trim(t) == what; };
      if (j >= in.size() || !is_open(in[j].text, "cond {")) return fail(ln, "stablehlo.while: expected 'cond {'");
      ++j;
      int nest = 0;
      for (; j < in.size(); ++j) {
        const std::string t = trim(in[j].text);
        if (nest == 0 && t == "} do {") break;
        if (!t.empty() && t.back() == '{') ++nest;
        if (!t.empty() && t[0] == '}') --nest;
        cond.push_back(in[j]);
      }
      if (j >= in.size()) return fail(ln, "stablehlo.while: expected '} do {'");
      ++j;
      nest = 0;
      for (; j < in.size(); ++j) {
        const std::string t = trim(in[j].text);
        if (nest == 0 && t == "}") break;
        if (!t.empty() && t.back() == '{') ++nest;
        if (!t.empty() && t[0] == '}') --nest;
        body.push_back(in[j]);
      }
      if (j >= in.size()) return fail(ln, "stablehlo.while: unterminated body");
      i = j;  // continue after the closing brace
      // ---- iterate
      std::vector<std::string> cur = init;  // SSA names (outer scope or renamed), or "" when only a constant is carried
      std::vector<bool> has_const(nres, false);
      std::vector<long long> cval(nres, 0);
      for (int k = 0; k < nres; ++k) {
        auto kn = known.find(init[k]);
        if (kn != known.end() && scalar_int_type(types[k])) {
          has_const[k] = true;
          cval[k] = kn->second;
        }
      }
      const int my = uid++;
      int trip = 0;
      while (true) {
        auto bind = [&](std::map<std::string, long long>& kn, std::map<std::string, std::string>& sb) {
          for (int k = 0; k < nres; ++k) {
            if (has_const[k]) kn[iter_names[k]] = cval[k];
            else kn.erase(iter_names[k]);
            sb[iter_names[k]] = cur[k];
          }
        };
        // condition: must fold to a constant
        {
          std::map<std::string, long long> kn = known;
          std::map<std::string, std::string> sb = sub;
          bind(kn, sb);
          // iteration-carried constants are referred to by the iter-arg names inside the regions
          for (int k = 0; k < nres; ++k)
            if (has_const[k]) sb.erase(iter_names[k]);
          std::vector<SrcLine> scratch;
          long long cv = 0;
          if (!eval_region(cond, kn, sb, scratch, depth, nullptr, &cv, true))
            return err.empty() ? fail(ln, "the condition of this while loop does not fold to a constant: only counted loops are unrolled") : false;
          if (!cv) break;
        }
        if (++trip > kMaxUnrollTrips) return fail(ln, "while loop with more than 64 trips is not unrolled");
        // body
        std::map<std::string, long long> kn = known;
        std::map<std::string, std::string> sb = sub;
        bind(kn, sb);
        for (int k = 0; k < nres; ++k)
          if (has_const[k]) sb.erase(iter_names[k]);
        // results defined inside the body get names unique to this trip
        for (auto& bl : body) {
          const std::string t = trim(bl.text);
          size_t e2 = t.find(" = ");
          if (t.empty() || t[0] != '%' || e2 == std::string::npos) continue;
          std::string r = trim(t.substr(0, e2));
          size_t c2 = r.find(':');
          if (c2 != std::string::npos) r = r.substr(0, c2);
          sb[r] = r + "_w" + std::to_string(my) + "_" + std::to_string(trip);
        }
        std::vector<std::string> yielded;
        if (!eval_region(body, kn, sb, out, depth, &yielded, nullptr, false)) return err.empty() ? fail(ln, "malformed while body") : false;
        if ((int)yielded.size() != nres) return fail(ln, "stablehlo.while: the body returns a different number of values");
        for (int k = 0; k < nres; ++k) {
          auto kv = kn.find(yielded[k]);
          if (kv != kn.end() && scalar_int_type(types[k])) {
            has_const[k] = true;
            cval[k] = kv->second;
            cur[k] = yielded[k];
          } else {
            has_const[k] = false;
            cur[k] = yielded[k];
          }
        }
      }
      // ---- results of the loop
      for (int k = 0; k < nres; ++k) {
        const std::string name = nres == 1 && colon == std::string::npos ? res : res + "#" + std::to_string(k);
        if (has_const[k]) {
          // a carried constant (the counter): give later users a constant op to read
          const std::string cname = res + "_w" + std::to_string(my) + "_c" + std::to_string(k);
          out.push_back({cname + " = stablehlo.constant dense<" + std::to_string(cval[k]) + "> : " + types[k], ln});
          known[cname] = cval[k];
          sub[name] = cname;
        } else {
          sub[name] = cur[k];
        }
      }
    }
    return true;
  }

  bool fail(int line, const std::string& what) {
    err = "line " + std::to_string(line) + ": " + what;
    return false;
  }

  // Runs the lines of a region.  Scalar integer ops whose operands are known are folded away; a
  // dynamic_slice with known indices becomes a slice; nested whiles are unrolled.  `yielded` receives the
  // operands of the terminating stablehlo.return; for a condition `*cond_value` receives its folded value.
  bool eval_region(const std::vector<SrcLine>& region, std::map<std::string, long long>& known,
                   std::map<std::string, std::string>& sub, std::vector<SrcLine>& out, int depth,
                   std::vector<std::string>* yielded, long long* cond_value, bool is_cond) {
    std::vector<SrcLine> ops;
    std::string ret;
    int ret_line = 0;
    for (auto& l : region) {
      const std::string t = trim(l.text);
      if (t.compare(0, 16, "stablehlo.return") == 0 || t.compare(0, 6, "return") == 0) {
        ret = t;
        ret_line = l.line;
        break;
      }
      ops.push_back(l);
    }
    std::vector<SrcLine> emitted;
    if (!run(ops, emitted, known, sub, depth + 1)) return false;
    if (is_cond) {
      for (auto& e : emitted)  // constants are kept as statements; anything else means the condition did not fold
        if (e.text.find("= stablehlo.constant ") == std::string::npos) return false;
    } else {
      out.insert(out.end(), emitted.begin(), emitted.end());
    }
    if (ret.empty()) return fail(region.empty() ? 0 : region[0].line, "region without stablehlo.return");
    size_t sp = ret.find(' ');
    std::string rest = sp == std::string::npos ? "" : ret.substr(sp + 1);
    size_t c = last_top_colon(rest);
    std::vector<std::string> vals = split_top(substitute(c == std::string::npos ? rest : rest.substr(0, c), sub));
    if (is_cond) {
      if (vals.size() != 1) return fail(ret_line, "a while condition returns one value");
      auto kv = known.find(vals[0]);
      if (kv == known.end()) return false;
      *cond_value = kv->second;
    } else if (yielded) {
      *yielded = vals;
    }
    return true;
  }

  // One non-while statement (already renamed): fold it if it is scalar integer arithmetic on known
  // values, rewrite dynamic_slice, otherwise pass it through.
  bool fold_or_emit(const std::string& l, int ln, std::vector<SrcLine>& out, std::map<std::string, long long>& known) {
    size_t eq = l.find(" = ");
    if (l.empty() || l[0] != '%' || eq == std::string::npos) {
      out.push_back({l, ln});
      return true;
    }
    const std::string res = trim(l.substr(0, eq));
    std::string rest = trim(l.substr(eq + 3));
    size_t c = last_top_colon(rest);
    if (c == std::string::npos) {
      out.push_back({l, ln});
      return true;
    }
    std::string head = trim(rest.substr(0, c)), sig = trim(rest.substr(c + 1));
    size_t sp = head.find_first_of(" (");
    std::string name = sp == std::string::npos ? head : head.substr(0, sp);
    std::string body = sp == std::string::npos ? "" : head.substr(sp);
    std::vector<std::string> operands;
    for (size_t i = 0; i < body.size(); ++i) {
      if (body[i] != '%') continue;
      size_t e = i + 1;
      while (e < body.size() && is_name_char(body[e])) ++e;
      operands.push_back(body.substr(i, e - i));
      i = e - 1;
    }
    std::string out_type = sig;
    size_t arrow = sig.find("->");
    if (arrow != std::string::npos) {
      out_type = trim(sig.substr(arrow + 2));
    } else {
      std::vector<std::string> ts = split_top(sig);  // "select" prints the predicate's type and the result's
      if (!ts.empty()) out_type = ts.back();
    }
    auto val = [&](size_t k, long long& v) {
      if (k >= operands.size()) return false;
      auto it = known.find(operands[k]);
      if (it == known.end()) return false;
      v = it->second;
      return true;
    };
    if (name == "stablehlo.constant" && scalar_int_type(out_type)) {
      size_t a = body.find("dense<"), b = body.rfind('>');
      if (a != std::string::npos && b != std::string::npos) {
        std::string v = trim(body.substr(a + 6, b - a - 6));
        if (v == "true") v = "1";
        if (v == "false") v = "0";
        if (!v.empty() && v.find_first_not_of("-0123456789") == std::string::npos) known[res] = atoll(v.c_str());
      }
      out.push_back({l, ln});  // kept: a later tensor op may read it
      return true;
    }
    if (scalar_int_type(out_type)) {
      long long x = 0, y = 0, z = 0;
      bool folded = false;
      long long r = 0;
      if (name == "stablehlo.compare" && val(0, x) && val(1, y)) {
        const std::string dir = body;
        folded = true;
        if (dir.find(" LT") != std::string::npos) r = x < y;
        else if (dir.find(" LE") != std::string::npos) r = x <= y;
        else if (dir.find(" GT") != std::string::npos) r = x > y;
        else if (dir.find(" GE") != std::string::npos) r = x >= y;
        else if (dir.find(" EQ") != std::string::npos) r = x == y;
        else if (dir.find(" NE") != std::string::npos) r = x != y;
        else folded = false;
      } else if ((name == "stablehlo.add" || name == "stablehlo.subtract" || name == "stablehlo.multiply" ||
                  name == "stablehlo.minimum" || name == "stablehlo.maximum" || name == "stablehlo.and" ||
                  name == "stablehlo.or") && val(0, x) && val(1, y)) {
        folded = true;
        r = name == "stablehlo.add" ? x + y : name == "stablehlo.subtract" ? x - y : name == "stablehlo.multiply" ? x * y
            : name == "stablehlo.minimum" ? std::min(x, y) : name == "stablehlo.maximum" ? std::max(x, y)
            : name == "stablehlo.and" ? (x & y) : (x | y);
      } else if (name == "stablehlo.select" && val(0, x) && val(1, y) && val(2, z)) {
        folded = true;
        r = x ? y : z;
      } else if (name == "stablehlo.clamp" && val(0, x) && val(1, y) && val(2, z)) {
        folded = true;
        r = std::min(std::max(y, x), z);
      } else if (name == "stablehlo.convert" && val(0, x)) {
        folded = true;
        r = x;
      }
      if (folded) {
        known[res] = r;
        return true;
      }
    }
    if (name == "stablehlo.dynamic_slice" && operands.size() >= 2) {
      std::vector<int64_t> sizes = int_list_after(body, "sizes");
      if (sizes.empty()) sizes = int_list_after(body, "slice_sizes");
      size_t p0 = sig.find('('), p1 = sig.find(')');
      std::vector<std::string> in_types = (p0 == std::string::npos || p1 == std::string::npos)
                                              ? std::vector<std::string>() : split_top(sig.substr(p0 + 1, p1 - p0 - 1));
      TType src = in_types.empty() ? TType() : parse_type(in_types[0]);
      bool all = src.ok && sizes.size() == src.dims.size() && operands.size() == src.dims.size() + 1;
      std::vector<long long> start(sizes.size(), 0);
      for (size_t k = 0; all && k < sizes.size(); ++k) {
        long long v;
        if (!val(k + 1, v)) all = false;
        else start[k] = std::min<long long>(std::max<long long>(v, 0), src.dims[k] - sizes[k]);  // clamped, as the op is defined
      }
      if (!all) return fail(ln, "dynamic_slice whose indices do not fold to constants is not supported");
      std::string lim;
      for (size_t k = 0; k < sizes.size(); ++k)
        lim += (k ? ", " : "") + std::to_string(start[k]) + ":" + std::to_string(start[k] + sizes[k]);
      out.push_back({res + " = stablehlo.slice " + operands[0] + " [" + lim + "] : (" + in_types[0] + ") -> " + out_type, ln});
      return true;
    }
    out.push_back({l, ln});
    return true;
  }
};

static bool parse_module(const char* text, size_t len, Module& m) {
  std::string all(text, len);
  std::vector<SrcLine> lines;
  {
    size_t p = 0;
    int n = 0;
    while (p <= all.size()) {
      size_t e = all.find('\n', p);
      if (e == std::string::npos) e = all.size();
      lines.push_back({all.substr(p, e - p), ++n});
      p = e + 1;
    }
  }
  if (all.find("stablehlo.while") != std::string::npos) {
    // counted loops are replaced by their bodies before anything else looks at the program
    Unroller u;
    std::vector<SrcLine> flat;
    std::map<std::string, long long> known;
    std::map<std::string, std::string> sub;
    if (!u.run(lines, flat, known, sub, 0)) {
      m.error = u.err.empty() ? "could not unroll a stablehlo.while loop" : u.err;
      return false;
    }
    lines.swap(flat);
  }
  bool in_main = false, seen_main = false;
  int lineno = 0;
  for (auto& src : lines) {
    lineno = src.line;
    const std::string& raw = src.text;
    std::string l = trim(raw);
    size_t loc = l.find(" loc(");
    if (loc != std::string::npos) l = trim(l.substr(0, loc));
    if (l.compare(0, 6, "module") == 0) {
      size_t at = l.find('@');
      if (at != std::string::npos) {
        size_t e = at + 1;
        while (e < l.size() && (isalnum((unsigned char)l[e]) || l[e] == '_' || l[e] == '.' || l[e] == '$')) ++e;
        if (e > at + 1) m.name = l.substr(at + 1, e - at - 1);
      }
      for (const char* key : {"mhlo.num_replicas", "mhlo.num_partitions"}) {
        size_t k = l.find(key);
        if (k == std::string::npos) continue;
        size_t eqs = l.find('=', k);
        if (eqs == std::string::npos) continue;
        const int v = atoi(l.c_str() + eqs + 1);
        if (v >= 1) (key[9] == 'r' ? m.num_replicas : m.num_partitions) = v;
      }
      continue;
    }
    if (l.empty() || l.compare(0, 2, "//") == 0 || l[0] == '#') continue;
    if (l.compare(0, 9, "func.func") == 0) {
      bool is_main = l.find("@main(") != std::string::npos;
      if (!is_main) {
        m.error = "line " + std::to_string(lineno) + ": only a single entry function @main is supported (found " +
                  l.substr(0, 60) + "...)";
        return false;
      }
      in_main = seen_main = true;
      size_t a = l.find("@main(") + 6;
      int depth = 1;
      size_t b = a;
      for (; b < l.size() && depth > 0; ++b) {
        if (l[b] == '(' || l[b] == '<' || l[b] == '{' || l[b] == '[') ++depth;
        if (l[b] == ')' || l[b] == '>' || l[b] == '}' || l[b] == ']') --depth;
        if (l[b] == '-' && b + 1 < l.size() && l[b + 1] == '>') ++b;
      }
      for (auto& a1 : split_top(l.substr(a, b - a - 1))) {
        size_t c = a1.find(':');
        if (c == std::string::npos) continue;
        std::string name = trim(a1.substr(0, c));
        std::string ty = trim(a1.substr(c + 1));
        size_t brace = ty.find(" {");
        if (brace != std::string::npos) ty = trim(ty.substr(0, brace));
        TType t = parse_type(ty);
        if (!t.ok) {
          m.error = "line " + std::to_string(lineno) + ": cannot read argument type '" + ty + "'";
          return false;
        }
        m.argi[name] = static_cast<int>(m.arg_names.size());
        m.arg_names.push_back(name);
        m.arg_types.push_back(t);
      }
      m.num_real_args = static_cast<int>(m.arg_names.size());
      continue;
    }
    if (!in_main) continue;
    if (l == "}") {
      in_main = false;
      continue;
    }
    if (l.compare(0, 6, "return") == 0 || l.compare(0, 11, "func.return") == 0) {
      size_t sp = l.find(' ');
      std::string rest = sp == std::string::npos ? "" : l.substr(sp + 1);
      size_t c = last_top_colon(rest);
      std::string vals = c == std::string::npos ? rest : rest.substr(0, c);
      for (auto& v : split_top(vals))
        if (!v.empty()) m.returns.push_back(v);
      continue;
    }
    // %name = op ...
    size_t eq = l.find(" = ");
    if (l[0] != '%' || eq == std::string::npos) {
      m.error = "line " + std::to_string(lineno) + ": unsupported statement '" + l.substr(0, 60) + "'";
      return false;
    }
    Op op;
    op.line = lineno;
    op.result = trim(l.substr(0, eq));
    if (op.result.find(':') != std::string::npos) {
      m.error = "line " + std::to_string(lineno) + ": multi-result ops are not supported";
      return false;
    }
    std::string rest = trim(l.substr(eq + 3));
    size_t c = last_top_colon(rest);
    if (c == std::string::npos) {
      m.error = "line " + std::to_string(lineno) + ": no type signature";
      return false;
    }
    std::string head = trim(rest.substr(0, c)), sig = trim(rest.substr(c + 1));
    // op name: stablehlo.xxx or "stablehlo.xxx"(...)
    if (head[0] == '"') {
      size_t e = head.find('"', 1);
      op.name = head.substr(1, e - 1);
      op.body = head.substr(e + 1);
    } else {
      size_t sp = head.find_first_of(" (");
      op.name = sp == std::string::npos ? head : head.substr(0, sp);
      op.body = sp == std::string::npos ? "" : head.substr(sp);
    }
    // operands: every %token of the body, in order
    for (size_t i = 0; i < op.body.size(); ++i) {
      if (op.body[i] != '%') continue;
      size_t e = i + 1;
      while (e < op.body.size() && (isalnum((unsigned char)op.body[e]) || op.body[e] == '_' || op.body[e] == '#')) ++e;
      op.operands.push_back(op.body.substr(i, e - i));
      i = e - 1;
    }
    // types
    size_t arrow = sig.find("->");
    if (arrow != std::string::npos && sig[0] == '(') {
      size_t close = sig.rfind(')', arrow);
      if (close == std::string::npos) {
        m.error = "line " + std::to_string(lineno) + ": malformed type signature of " + op.name;
        return false;
      }
      for (auto& t : split_top(sig.substr(1, close - 1))) op.in_types.push_back(parse_type(t));
      op.out_type = parse_type(sig.substr(arrow + 2));
    } else {
      op.out_type = parse_type(sig);
      for (size_t i = 0; i < op.operands.size(); ++i) op.in_types.push_back(op.out_type);
    }
    if (!op.out_type.ok) {
      m.error = "line " + std::to_string(lineno) + ": cannot read result type of " + op.name;
      return false;
    }
    if (op.name == "stablehlo.constant") {
      std::vector<uint8_t> bytes;
      std::string err;
      const int kind = parse_dense(op.body, op.out_type, bytes, err);
      if (kind < 0) {
        m.error = "line " + std::to_string(lineno) + ": " + err;
        return false;
      }
      if (kind == 1) {
        // a dense constant (a weight closed over by the function): treated from here on as one
        // more argument of @main whose buffer the plan owns
        m.argi[op.result] = static_cast<int>(m.arg_names.size());
        m.arg_names.push_back(op.result);
        m.arg_types.push_back(op.out_type);
        m.const_data.push_back(std::move(bytes));
        continue;
      }
    }
    m.def[op.result] = static_cast<int>(m.ops.size());
    m.ops.push_back(op);
  }
  if (!seen_main) {
    m.error = "no func.func @main found";
    return false;
  }
  return true;
}

// ---------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------
enum StepKind { kW8A32 = 0, kW8A16 = 1, kI8Dot = 2, kW4A16 = 3, kGeneric = 4 };
enum GenericOp { gConvert = 0, gBinary, gGather, gConcat, gFill, gDot, gCopy };

// Operands and results of a step are value slots: [0, A) the arguments of @main (lifted constants
// included), [A, A + R) its results, above that temporaries inside the plan's workspace.
struct Step {
  StepKind kind;
  int64_t M = 0, N = 0, K = 0;
  int x = -1, w = -1, scale = -1, zeros = -1, row = -1, col = -1;
  int out = -1, acc_out = -1;  // -1 = not produced
  int a_unsigned = 0, b_unsigned = 0, zeros_packed = 0;
  int anchor_line = 0;
  int anchor_op = 0;  // index of the op the step stands for (steps run in this order)
  int fused_ops = 0;
  // how the fused kernel's arithmetic relates to the program as written: "as_written", or what differs
  const char* numerics = "as_written";
  // standalone ops
  int gop = 0, bop = 0, in_dt = 0, out_dt = 0, b_transposed = 0;
  std::vector<int> ins;
  long long count = 0;
  std::vector<long long> in_dims, out_dims, src_of, start, stride;  // gather
  long long outer = 1, inner = 1, out_len = 0;                        // concatenate
  std::vector<long long> part_len;
  double fval = 0;
  long long ival = 0;
  size_t bytes = 0;  // copy
};

struct Plan {
  Module mod;
  std::vector<Step> steps;
  std::string trace;  // JSON lines
  size_t scratch = 0;    // kernel scratch (the int4 decode kernel's), at the start of the workspace
  size_t workspace = 0;  // scratch + temporaries
  std::map<std::string, int> slot;     // SSA value -> slot
  std::vector<size_t> temp_offset;     // per temporary, from the start of the workspace
  // device copies of the lifted constants, per device ordinal (created on first execution there)
  std::mutex mu;
  std::map<int, std::vector<void*>> const_dev;
};

// A value seen as "argument A with its dimensions placed on some dimensions of
// the current tensor, all other dimensions broadcast".  Follows
// broadcast_in_dim / reshape (size-1 insertions only) / convert back to an
// argument.  dim_of[i] = source dimension feeding result dimension i, or -1.
struct View {
  int arg = -1;
  std::vector<int> dim_of;
  std::vector<int> ops;  // op indices walked through
  bool converted = false;
};

static bool view_of(const Module& m, const std::string& v, View& out) {
  auto a = m.argi.find(v);
  if (a != m.argi.end()) {
    out.arg = a->second;
    out.dim_of.clear();
    for (size_t i = 0; i < m.arg_types[a->second].dims.size(); ++i) out.dim_of.push_back((int)i);
    return true;
  }
  auto d = m.def.find(v);
  if (d == m.def.end()) return false;
  const Op& op = m.ops[d->second];
  if (op.operands.size() != 1) return false;
  View in;
  if (!view_of(m, op.operands[0], in)) return false;
  const TType& it = op.in_types.empty() ? TType() : op.in_types[0];
  const TType& ot = op.out_type;
  out = in;
  out.ops.push_back(d->second);
  if (op.name == "stablehlo.convert") {
    out.converted = true;
    return true;
  }
  if (op.name == "stablehlo.broadcast_in_dim") {
    std::vector<int64_t> dims = int_list_after(op.body, "dims");
    if (dims.size() != it.dims.size()) return false;
    out.dim_of.assign(ot.dims.size(), -1);
    for (size_t i = 0; i < dims.size(); ++i) {
      if (dims[i] < 0 || dims[i] >= (int64_t)ot.dims.size()) return false;
      if (it.dims[i] == ot.dims[dims[i]] && in.dim_of[i] >= 0) out.dim_of[dims[i]] = in.dim_of[i];
      else if (it.dims[i] != 1 && it.dims[i] != ot.dims[dims[i]]) return false;
    }
    return true;
  }
  if (op.name == "stablehlo.reshape") {
    // only insertion/removal of size-1 dimensions
    std::vector<int> src;
    for (size_t i = 0; i < it.dims.size(); ++i)
      if (it.dims[i] != 1) src.push_back((int)i);
    out.dim_of.assign(ot.dims.size(), -1);
    size_t k = 0;
    for (size_t i = 0; i < ot.dims.size(); ++i) {
      if (ot.dims[i] == 1) continue;
      if (k >= src.size() || it.dims[src[k]] != ot.dims[i]) return false;
      out.dim_of[i] = in.dim_of[src[k]];
      ++k;
    }
    return k == src.size();
  }
  return false;
}

static const Op* def_of(const Module& m, const std::string& v, int* idx = nullptr) {
  auto d = m.def.find(v);
  if (d == m.def.end()) return nullptr;
  if (idx) *idx = d->second;
  return &m.ops[d->second];
}

static bool is_splat_const(const Module& m, const std::string& v, long long want, std::vector<int>* used) {
  int idx;
  const Op* op = def_of(m, v, &idx);
  if (!op) return false;
  if (op->name == "stablehlo.broadcast_in_dim" && op->operands.size() == 1) {
    used->push_back(idx);
    return is_splat_const(m, op->operands[0], want, used);
  }
  if (op->name != "stablehlo.constant") return false;
  size_t a = op->body.find("dense<");
  if (a == std::string::npos) return false;
  size_t b = op->body.find('>', a);
  std::string val = trim(op->body.substr(a + 6, b - a - 6));
  if (val.empty() || val[0] == '[') return false;
  used->push_back(idx);
  return atoll(val.c_str()) == want;
}

static void tracef(std::string& t, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  t += "QMM_PLAN_JSON:";
  t += buf;
  t += "\n";
}

static int result_index(const Module& m, const std::string& v) {
  for (size_t i = 0; i < m.returns.size(); ++i)
    if (m.returns[i] == v) return (int)i;
  return -1;
}

static bool is_float(const std::string& e) { return e == "f32" || e == "bf16" || e == "f16"; }

// nibble planes of a packed [K/2, N] byte argument interleaved along K:
//   reshape(concatenate(dim=1)(view(and(Wq,15)), view(shift_right_logical(Wq,4)))) : [K/2,2,N] -> [K,N] (or [G,g,N])
static bool match_unpack4(const Module& m, const std::string& v, int* warg, std::vector<int>* used) {
  int idx;
  const Op* rs = def_of(m, v, &idx);
  if (!rs) return false;
  const Op* cat = rs;
  if (rs->name == "stablehlo.reshape") {
    used->push_back(idx);
    cat = def_of(m, rs->operands[0], &idx);
    if (!cat) return false;
  }
  if (cat->name != "stablehlo.concatenate" || cat->operands.size() != 2) return false;
  used->push_back(idx);
  size_t p = cat->body.find("dim");
  if (p == std::string::npos) return false;
  size_t e = cat->body.find('=', p);
  if (e == std::string::npos || atoll(cat->body.c_str() + e + 1) != 1) return false;
  if (cat->out_type.dims.size() != 3 || cat->out_type.dims[1] != 2) return false;
  int args[2] = {-1, -1};
  for (int half = 0; half < 2; ++half) {
    // walk size-1 reshapes / broadcasts down to the and / shift op
    std::string cur = cat->operands[half];
    const Op* o = nullptr;
    for (int hop = 0; hop < 4; ++hop) {
      o = def_of(m, cur, &idx);
      if (!o) return false;
      if ((o->name == "stablehlo.reshape" || o->name == "stablehlo.broadcast_in_dim") && o->operands.size() == 1 &&
          o->out_type.count() == o->in_types[0].count()) {
        used->push_back(idx);
        cur = o->operands[0];
        continue;
      }
      break;
    }
    const char* want = half == 0 ? "stablehlo.and" : "stablehlo.shift_right_logical";
    if (!o || o->name != want || o->operands.size() != 2) return false;
    used->push_back(idx);
    int ai = -1;
    std::string cst;
    for (int k = 0; k < 2; ++k) {
      auto a = m.argi.find(o->operands[k]);
      if (a != m.argi.end()) ai = a->second;
      else cst = o->operands[k];
    }
    if (ai < 0 || cst.empty()) return false;
    if (!is_splat_const(m, cst, half == 0 ? 15 : 4, used)) return false;
    args[half] = ai;
  }
  if (args[0] != args[1]) return false;
  const TType& wt = m.arg_types[args[0]];
  if (wt.dims.size() != 2 || (wt.elem != "ui8" && wt.elem != "i8")) return false;
  *warg = args[0];
  return true;
}

// Slices of an argument that select one contiguous block (unit strides; full extent in every
// dimension after the first partial one, extent 1 before it) and reshapes of arguments become
// arguments themselves that point into their source: a scan over stacked [layers, K, N] weights then
// hands the matcher one [K, N] "argument" per layer without copying anything.
static void lift_argument_views(Module& m) {
  for (size_t i = 0; i < m.ops.size(); ++i) {
    const Op& op = m.ops[i];
    if (op.operands.size() != 1 || op.in_types.empty()) continue;
    auto src = m.argi.find(op.operands[0]);
    if (src == m.argi.end()) continue;
    const TType& it = op.in_types[0];
    const TType& ot = op.out_type;
    const size_t bits = gen::dtype_bits(dtype_of_elem_early(it.elem));
    if (bits < 8 || it.elem != ot.elem) continue;
    size_t offset = 0;
    if (op.name == "stablehlo.reshape") {
      // only reshapes of a slice view (dropping its unit dimensions); reshapes of plain arguments stay
      // ops, which the matchers read through
      if (it.count() != ot.count() || src->second < m.num_real_args + (int)m.const_data.size()) continue;
    } else if (op.name == "stablehlo.slice") {
      size_t a = op.body.find('['), b = op.body.find(']');
      if (a == std::string::npos || b == std::string::npos) continue;
      std::vector<std::string> parts = split_top(op.body.substr(a + 1, b - a - 1));
      if (parts.size() != it.dims.size() || ot.dims.size() != it.dims.size()) continue;
      bool ok = true;
      int64_t stride = 1;
      std::vector<int64_t> start(parts.size());
      for (size_t d = 0; d < parts.size(); ++d) {
        size_t c1 = parts[d].find(':');
        if (c1 == std::string::npos) { ok = false; break; }
        size_t c2 = parts[d].find(':', c1 + 1);
        start[d] = atoll(parts[d].c_str());
        const int64_t limit = atoll(parts[d].c_str() + c1 + 1);
        const int64_t step = c2 == std::string::npos ? 1 : atoll(parts[d].c_str() + c2 + 1);
        if (step != 1 || limit - start[d] != ot.dims[d] || start[d] < 0 || limit > it.dims[d]) { ok = false; break; }
      }
      if (!ok) continue;
      // contiguity: before the first dimension with extent > 1 everything has extent 1; after it, full extent
      size_t first_wide = 0;
      while (first_wide < parts.size() && ot.dims[first_wide] == 1) ++first_wide;
      for (size_t d = first_wide + 1; d < parts.size(); ++d)
        if (ot.dims[d] != it.dims[d]) ok = false;
      if (!ok) continue;
      for (int d = (int)parts.size() - 1; d >= 0; --d) {
        offset += (size_t)(start[d] * stride) * bits / 8;
        stride *= it.dims[d];
      }
    } else {
      continue;
    }
    // the source may itself be a view: offsets add up on the original argument
    int base = src->second;
    const int first_view = m.num_real_args + (int)m.const_data.size();
    if (base >= first_view) {
      offset += m.views[base - first_view].second;
      base = m.views[base - first_view].first;
    }
    m.argi[op.result] = (int)m.arg_names.size();
    m.arg_names.push_back(op.result);
    m.arg_types.push_back(ot);
    m.views.push_back({base, offset});
    m.view_ops.insert((int)i);
  }
}

// ---------------------------------------------------------------------------
// Explicit route: stablehlo.custom_call @qmm_b200.qmm with a JSON backend_config.
// A guaranteed-fused entry that does not depend on the matcher recognising a jnp spelling; the
// mechanism follows the reference's native-kernel custom call (src/jax_plugins/silicon/
// _native_metal.py:34-60,179-196, dispatched in src/pjrt_plugin/ops/control_flow_ops.mm:1194-1222),
// and its conventions for the descriptor (runtime/custom_metal_kernel.mm:129-193): versioned JSON,
// exact-key validation, a size limit.
//   {"version":1,"op":"w8a32_perchannel"}          operands (x f32, w i8, scale f32)      -> f32
//   {"version":1,"op":"w8a16_perchannel"}          operands (x bf16, w i8, scale f32)     -> bf16
//   {"version":1,"op":"i8i8_i32"}                  operands (a, b) -> i32, or (a, b, row, col) -> f32
//   {"version":1,"op":"w4a16_g128","zeros_packed":true|false}
//                                                  operands (x bf16, wq u8, scales bf16, zeros) -> bf16
// ---------------------------------------------------------------------------
constexpr const char* kCustomCallTarget = "qmm_b200.qmm";

// A flat JSON object of string / integer / boolean values.  Returns false with `err` set.
static bool parse_flat_json(const std::string& j, std::map<std::string, std::string>& out, std::string& err) {
  size_t i = 0;
  auto ws = [&] { while (i < j.size() && (j[i] == ' ' || j[i] == '\t' || j[i] == '\n')) ++i; };
  auto str = [&](std::string& v) -> bool {
    if (i >= j.size() || j[i] != '"') return false;
    ++i;
    v.clear();
    while (i < j.size() && j[i] != '"') {
      if (j[i] == '\\') return false;  // no escapes inside this descriptor's strings
      v += j[i++];
    }
    if (i >= j.size()) return false;
    ++i;
    return true;
  };
  ws();
  if (i >= j.size() || j[i] != '{') { err = "backend_config must be a JSON object"; return false; }
  ++i;
  ws();
  if (i < j.size() && j[i] == '}') return true;
  while (true) {
    std::string k, v;
    ws();
    if (!str(k)) { err = "invalid backend_config JSON: expected a key"; return false; }
    ws();
    if (i >= j.size() || j[i] != ':') { err = "invalid backend_config JSON: expected ':'"; return false; }
    ++i;
    ws();
    if (i < j.size() && j[i] == '"') {
      if (!str(v)) { err = "invalid backend_config JSON: bad string"; return false; }
      v = "s:" + v;
    } else {
      size_t b = i;
      while (i < j.size() && j[i] != ',' && j[i] != '}' && j[i] != ' ') ++i;
      v = j.substr(b, i - b);
      if (v != "true" && v != "false" && (v.empty() || v.find_first_not_of("-0123456789") != std::string::npos)) {
        err = "invalid backend_config JSON: value of '" + k + "' must be a string, an integer or a boolean";
        return false;
      }
    }
    if (out.count(k)) { err = "backend_config repeats the key '" + k + "'"; return false; }
    out[k] = v;
    ws();
    if (i < j.size() && j[i] == ',') { ++i; continue; }
    if (i < j.size() && j[i] == '}') { ++i; break; }
    err = "invalid backend_config JSON: expected ',' or '}'";
    return false;
  }
  ws();
  if (i != j.size()) { err = "invalid backend_config JSON: trailing characters"; return false; }
  return true;
}

static int build_plan(Plan& plan) {
  Module& m = plan.mod;
  const int A = (int)m.arg_names.size(), R = (int)m.returns.size();
  std::set<int> consumed = m.view_ops;  // ops absorbed into a fused step (views of arguments move no data)
  // users of every value, to make sure absorbed intermediates do not escape
  std::map<std::string, std::vector<int>> users;
  for (size_t i = 0; i < m.ops.size(); ++i)
    for (auto& o : m.ops[i].operands) users[o].push_back((int)i);

  // slot of a value: argument, result (its first position in the return list) or a new temporary
  auto type_of = [&](const std::string& v) -> const TType* {
    auto a = m.argi.find(v);
    if (a != m.argi.end()) return &m.arg_types[a->second];
    auto d = m.def.find(v);
    return d == m.def.end() ? nullptr : &m.ops[d->second].out_type;
  };
  std::vector<size_t> temp_bytes;
  auto slot_of = [&](const std::string& v) -> int {
    auto it = plan.slot.find(v);
    if (it != plan.slot.end()) return it->second;
    int sl;
    auto a = m.argi.find(v);
    const int r = result_index(m, v);
    if (a != m.argi.end()) sl = a->second;
    else if (r >= 0) sl = A + r;
    else {
      const TType* t = type_of(v);
      const size_t bits = t ? gen::dtype_bits(dtype_of_elem_early(t->elem)) : 0;
      sl = A + R + (int)temp_bytes.size();
      temp_bytes.push_back(t ? ((size_t)t->count() * bits / 8 + 255) / 256 * 256 : 0);
    }
    plan.slot[v] = sl;
    return sl;
  };

  // ---- one dot: try the fused patterns.  QMM_ERR_UNSUPPORTED = "not a pattern this backend fuses"
  // (the dot then runs unfused); any other error is final.
  auto match = [&](size_t di, Step& st, std::vector<int>& used) -> int {
    const Op& dot = m.ops[di];
    if (dot.operands.size() != 2 || dot.in_types.size() != 2)
      return set_error(QMM_ERR_PARSE, "line %d: malformed %s", dot.line, dot.name.c_str());
    const TType &lt = dot.in_types[0], &rt = dot.in_types[1], &ot = dot.out_type;
    std::vector<int64_t> lc, rc, lb;
    if (dot.name == "stablehlo.dot_general") {
      size_t e = 0;
      lb = int_list_after(dot.body, "batching_dims");
      lc = int_list_after(dot.body, "contracting_dims", 0, &e);
      if (!lc.empty()) rc = int_list_after(dot.body, "x", e);
      if (lc.empty()) {  // generic attribute spelling
        lc = int_list_after(dot.body, "lhs_contracting_dimensions");
        rc = int_list_after(dot.body, "rhs_contracting_dimensions");
        lb = int_list_after(dot.body, "lhs_batching_dimensions");
      }
    } else {
      lc = {(int64_t)lt.dims.size() - 1};
      rc = {0};
    }
    if (!lb.empty() || lc.size() != 1 || rc.size() != 1 || rt.dims.size() != 2 || rc[0] != 0 ||
        lc[0] != (int64_t)lt.dims.size() - 1 || lt.dims.empty())
      return set_error(QMM_ERR_UNSUPPORTED,
                       "line %d: %s with these dimension numbers is not on the quantized-matmul path "
                       "(need [...,K] x [K,N], no batch dimensions)",
                       dot.line, dot.name.c_str());
    const int64_t K = rt.dims[0], N = rt.dims[1];
    int64_t M = 1;
    for (size_t i = 0; i + 1 < lt.dims.size(); ++i) M *= lt.dims[i];
    if (lt.dims.back() != K)
      return set_error(QMM_ERR_PARSE, "line %d: contracting sizes differ", dot.line);
    st.M = M; st.N = N; st.K = K;
    st.anchor_line = dot.line;
    st.anchor_op = (int)di;
    used.push_back((int)di);

    auto lhs_arg = m.argi.find(dot.operands[0]);
    const bool int_dot = (lt.elem == "i8" || lt.elem == "ui8") && (rt.elem == "i8" || rt.elem == "ui8");
    if (int_dot) {
      // ---- P2 ----
      auto rhs_arg = m.argi.find(dot.operands[1]);
      if (lhs_arg == m.argi.end() || rhs_arg == m.argi.end() || ot.elem != "i32")
        return set_error(QMM_ERR_UNSUPPORTED,
                         "line %d: integer dot_general must take two int8/uint8 arguments and produce i32 "
                         "(preferred_element_type=int32)", dot.line);
      st.kind = kI8Dot;
      st.x = lhs_arg->second;
      st.w = rhs_arg->second;
      st.a_unsigned = lt.elem == "ui8";
      st.b_unsigned = rt.elem == "ui8";
      // optional rescale chain: convert -> multiply(row) -> multiply(col), either order
      std::string cur = dot.result;
      int got_row = -1, got_col = -1;
      std::string last = "";
      std::vector<int> chain;
      auto single_user = [&](const std::string& v, const char* name) -> int {
        int found = -1;
        for (int u : users[v])
          if (m.ops[u].name == name) found = found < 0 ? u : -2;
        return found;
      };
      int cv = single_user(cur, "stablehlo.convert");
      if (cv >= 0 && m.ops[cv].out_type.elem == "f32") {
        chain.push_back(cv);
        cur = m.ops[cv].result;
        for (int hop = 0; hop < 2; ++hop) {
          int mu = single_user(cur, "stablehlo.multiply");
          if (mu < 0) break;
          const Op& mul = m.ops[mu];
          std::string other = mul.operands[0] == cur ? mul.operands[1] : mul.operands[0];
          View v;
          if (!view_of(m, other, v) || v.dim_of.size() != 2) break;
          const TType& at = m.arg_types[v.arg];
          if (at.elem != "f32" || at.dims.size() != 1) break;
          if (v.dim_of[0] == 0 && v.dim_of[1] == -1 && at.dims[0] == M && got_row < 0) {
            got_row = v.arg;
          } else if (v.dim_of[0] == -1 && v.dim_of[1] == 0 && at.dims[0] == N && got_col < 0) {
            got_col = v.arg;
            if (got_row < 0) st.numerics = "rescale_reordered: the kernel multiplies by the row scale first";
          }
          else break;
          chain.push_back(mu);
          for (int o : v.ops) chain.push_back(o);
          cur = mul.result;
          last = cur;
        }
      }
      if (got_row >= 0 && got_col >= 0) {
        // the order convert -> row -> col is what the kernel's epilogue computes; col -> row differs
        // only by f32 rounding of one product and is accepted as the same fused step
        st.row = got_row;
        st.col = got_col;
        st.out = slot_of(last);
        for (int o : chain) used.push_back(o);
      }
      {
        // the int32 accumulator itself is needed when it is returned or read by an op outside the chain
        std::set<int> in_chain(used.begin(), used.end());
        bool need_acc = result_index(m, dot.result) >= 0 || st.out < 0;
        for (int u : users[dot.result])
          if (!in_chain.count(u)) need_acc = true;
        if (need_acc) st.acc_out = slot_of(dot.result);
      }
    } else if (is_float(lt.elem)) {
      st.x = slot_of(dot.operands[0]);
      // rhs chain
      int ri;
      const Op* r = def_of(m, dot.operands[1], &ri);
      if (!r)
        return set_error(QMM_ERR_UNSUPPORTED,
                         "line %d: plain float dot_general (no dequantisation chain feeds it)",
                         dot.line);
      const Op* top = r;
      if (top->name == "stablehlo.reshape" && top->in_types[0].dims.size() == 3) {
        // ---- P3: reshape([G,g,N] -> [K,N]) of (q - z) * s ----
        used.push_back(ri);
        const TType& g3 = top->in_types[0];
        const int64_t G = g3.dims[0], gs = g3.dims[1];
        if (g3.dims[2] != N || G * gs != K)
          return set_error(QMM_ERR_PARSE, "line %d: group reshape does not match the dot", top->line);
        int mi;
        const Op* mul = def_of(m, top->operands[0], &mi);
        if (!mul || mul->name != "stablehlo.multiply")
          return set_error(QMM_ERR_UNSUPPORTED, "line %d: expected multiply by group scales before %s",
                           top->line, "stablehlo.reshape");
        used.push_back(mi);
        View sv;
        std::string subv;
        for (int k = 0; k < 2; ++k) {
          View v;
          if (view_of(m, mul->operands[k], v) && v.dim_of.size() == 3 && v.dim_of[0] == 0 && v.dim_of[1] == -1 &&
              v.dim_of[2] == 1) {
            sv = v;
            subv = mul->operands[1 - k];
          }
        }
        if (sv.arg < 0 || m.arg_types[sv.arg].elem != "bf16" || sv.converted)
          return set_error(QMM_ERR_UNSUPPORTED,
                           "line %d: group scales must be a bf16 [K/g, N] argument broadcast on dims [0, 2]",
                           mul->line);
        for (int o : sv.ops) used.push_back(o);
        int si;
        const Op* sub = def_of(m, subv, &si);
        if (!sub || sub->name != "stablehlo.subtract")
          return set_error(QMM_ERR_UNSUPPORTED, "line %d: expected subtract of zero points", mul->line);
        used.push_back(si);
        View zv;
        if (!view_of(m, sub->operands[1], zv) || zv.dim_of.size() != 3 || zv.dim_of[0] != 0 || zv.dim_of[1] != -1 ||
            zv.dim_of[2] != 1)
          return set_error(QMM_ERR_UNSUPPORTED,
                           "line %d: zero points must be a [K/g, N] argument broadcast on dims [0, 2]", sub->line);
        for (int o : zv.ops) used.push_back(o);
        const TType& zt = m.arg_types[zv.arg];
        if (zt.elem != "ui4" && zt.elem != "ui8" && zt.elem != "i8")
          return set_error(QMM_ERR_UNSUPPORTED, "line %d: zero points must be ui4 or ui8, got %s", sub->line,
                           zt.elem.c_str());
        // q: convert(unpack) possibly reshaped to [G,g,N]
        std::string qv = sub->operands[0];
        int warg = -1;
        for (int hop = 0; hop < 3 && warg < 0; ++hop) {
          int qi;
          const Op* q = def_of(m, qv, &qi);
          if (!q) break;
          if (q->name == "stablehlo.convert" ||
              (q->name == "stablehlo.reshape" && q->in_types[0].dims.size() == 2)) {
            used.push_back(qi);
            qv = q->operands[0];
            std::vector<int> u2;
            if (match_unpack4(m, qv, &warg, &u2)) {
              for (int o : u2) used.push_back(o);
            }
            continue;
          }
          break;
        }
        if (warg < 0)
          return set_error(QMM_ERR_UNSUPPORTED,
                           "line %d: could not recognise the int4 unpack (and 15 / shift_right_logical 4 / "
                           "concatenate dim 1) feeding the subtract", sub->line);
        const TType& wt = m.arg_types[warg];
        if (wt.dims[0] * 2 != K || wt.dims[1] != N)
          return set_error(QMM_ERR_PARSE, "line %d: packed weight shape does not match the dot", dot.line);
        if (gs != 128 || lt.elem != "bf16" || ot.elem != "bf16")
          return set_error(QMM_ERR_UNSUPPORTED,
                           "line %d: the int4 kernel covers group 128 with bf16 activations and result "
                           "(got group %lld, %s -> %s)", dot.line, (long long)gs, lt.elem.c_str(), ot.elem.c_str());
        st.kind = kW4A16;
        st.numerics = M <= 32 ? "f32_group_sums: (q - z) * s applied per 128-k group to f32 sums, not rounded to bf16 per weight"
                              : "as_written";
        st.w = warg;
        st.scale = sv.arg;
        st.zeros = zv.arg;
        st.zeros_packed = zt.elem == "ui4";  // 4-bit buffers hold two values per byte, low nibble first
        st.out = slot_of(dot.result);
      } else if (top->name == "stablehlo.multiply") {
        // ---- P1: convert(W:i8) * broadcast(scale) ----
        used.push_back(ri);
        int warg = -1;
        View sv;
        for (int k = 0; k < 2; ++k) {
          int ci;
          const Op* cv = def_of(m, top->operands[k], &ci);
          auto wa = cv && cv->name == "stablehlo.convert" && cv->operands.size() == 1
                        ? m.argi.find(cv->operands[0]) : m.argi.end();
          View v;
          if (wa != m.argi.end() && m.arg_types[wa->second].elem == "i8" && view_of(m, top->operands[1 - k], v) &&
              v.dim_of.size() == 2 && v.dim_of[0] == -1 && v.dim_of[1] == 0) {
            warg = wa->second;
            sv = v;
            used.push_back(ci);
          }
        }
        if (warg < 0)
          return set_error(QMM_ERR_UNSUPPORTED,
                           "line %d: expected convert(int8 weight) * broadcast(per-channel scale) as the rhs of "
                           "the dot on line %d", top->line, dot.line);
        for (int o : sv.ops) used.push_back(o);
        const TType& st_t = m.arg_types[sv.arg];
        if (st_t.elem != "f32" || st_t.dims.size() != 1 || st_t.dims[0] != N)
          return set_error(QMM_ERR_UNSUPPORTED, "line %d: the per-channel scale must be an f32 [N] argument",
                           top->line);
        std::string outv = dot.result;
        if (lt.elem == "f32" && ot.elem == "f32") st.kind = kW8A32;
        else if (lt.elem == "bf16" && ot.elem == "bf16") st.kind = kW8A16;
        else if (lt.elem == "bf16" && ot.elem == "f32" && users[dot.result].size() == 1 &&
                 result_index(m, dot.result) < 0 && m.ops[users[dot.result][0]].name == "stablehlo.convert" &&
                 m.ops[users[dot.result][0]].out_type.elem == "bf16") {
          // bf16 operands, f32 result (preferred_element_type) rounded to bf16 by a convert: the
          // kernel accumulates in f32 and rounds once, which is exactly this
          st.kind = kW8A16;
          used.push_back(users[dot.result][0]);
          outv = m.ops[users[dot.result][0]].result;
        } else
          return set_error(QMM_ERR_UNSUPPORTED, "line %d: %s activations with %s result are not covered",
                           dot.line, lt.elem.c_str(), ot.elem.c_str());
        if (lt.elem == "bf16")
          st.numerics = "f32_scale_in_epilogue: the scale stays f32 and multiplies the f32 accumulator once; the program "
                        "rounds the scale and every w * s product to bf16";
        st.w = warg;
        st.scale = sv.arg;
        st.out = slot_of(outv);
      } else {
        return set_error(QMM_ERR_UNSUPPORTED,
                         "line %d: the rhs of the dot on line %d is produced by %s, which is not a dequantisation "
                         "chain this backend fuses", top->line, dot.line, top->name.c_str());
      }
    } else {
      return set_error(QMM_ERR_UNSUPPORTED,
                       "line %d: dot_general with %s x %s operands is not on the quantized-matmul path", dot.line,
                       lt.elem.c_str(), rt.elem.c_str());
    }
    return QMM_OK;
  };

  // ---- explicit custom calls
  for (size_t ci = 0; ci < m.ops.size(); ++ci) {
    const Op& op = m.ops[ci];
    if (op.name != "stablehlo.custom_call") continue;
    size_t at = op.body.find('@');
    size_t par = at == std::string::npos ? std::string::npos : op.body.find('(', at);
    const std::string target = par == std::string::npos ? "" : trim(op.body.substr(at + 1, par - at - 1));
    if (target != kCustomCallTarget)
      return set_error(QMM_ERR_UNSUPPORTED, "line %d: custom_call target '%s' is not one this backend executes (only @%s)",
                       op.line, target.c_str(), kCustomCallTarget);
    size_t bc = op.body.find("backend_config");
    size_t q0 = bc == std::string::npos ? std::string::npos : op.body.find('"', bc);
    if (q0 == std::string::npos) return set_error(QMM_ERR_PARSE, "line %d: custom_call without a backend_config string", op.line);
    std::string json;
    size_t q = q0 + 1;
    for (; q < op.body.size() && op.body[q] != '"'; ++q) {
      if (op.body[q] == '\\' && q + 1 < op.body.size()) json += op.body[++q];  // \" inside the MLIR string attribute
      else json += op.body[q];
    }
    if (q >= op.body.size()) return set_error(QMM_ERR_PARSE, "line %d: unterminated backend_config", op.line);
    if (json.size() > 4096) return set_error(QMM_ERR_INVALID_ARGUMENT, "line %d: backend_config larger than 4096 bytes", op.line);
    std::map<std::string, std::string> cfg;
    std::string jerr;
    if (!parse_flat_json(json, cfg, jerr)) return set_error(QMM_ERR_INVALID_ARGUMENT, "line %d: %s", op.line, jerr.c_str());
    if (!cfg.count("version") || !cfg.count("op"))
      return set_error(QMM_ERR_INVALID_ARGUMENT, "line %d: backend_config needs the keys \"version\" and \"op\"", op.line);
    if (cfg["version"] != "1")
      return set_error(QMM_ERR_INVALID_ARGUMENT, "line %d: unsupported backend_config version (expected 1)", op.line);
    const std::string kind = cfg["op"].compare(0, 2, "s:") == 0 ? cfg["op"].substr(2) : "";
    for (auto& kv : cfg) {
      const bool known = kv.first == "version" || kv.first == "op" || (kind == "w4a16_g128" && kv.first == "zeros_packed");
      if (!known)
        return set_error(QMM_ERR_INVALID_ARGUMENT, "line %d: backend_config has the unknown key \"%s\"", op.line, kv.first.c_str());
    }
    Step st;
    st.anchor_line = op.line;
    st.anchor_op = (int)ci;
    const size_t no = op.operands.size();
    auto elem = [&](size_t k) { return k < op.in_types.size() ? op.in_types[k].elem : std::string(); };
    auto dims = [&](size_t k) -> const std::vector<int64_t>& { return op.in_types[k].dims; };
    const TType& ot = op.out_type;
    auto bad = [&](const char* what) {
      return set_error(QMM_ERR_INVALID_ARGUMENT, "line %d: custom_call @%s op \"%s\": %s", op.line, kCustomCallTarget,
                       kind.c_str(), what);
    };
    if (op.in_types.size() != no || no < 2 || dims(0).size() != 2 || dims(1).size() != 2 || ot.dims.size() != 2)
      return bad("operands and result must be rank-2 tensors with a full type signature");
    st.M = dims(0)[0];
    st.N = ot.dims[1];
    if (kind == "w8a32_perchannel" || kind == "w8a16_perchannel") {
      const bool f32 = kind == "w8a32_perchannel";
      if (no != 3 || elem(0) != (f32 ? "f32" : "bf16") || elem(1) != "i8" || elem(2) != "f32" || ot.elem != elem(0))
        return bad("expects (x, w: i8, scale: f32) with x and the result f32 (w8a32) or bf16 (w8a16)");
      st.K = dims(0)[1];
      if (dims(1)[0] != st.K || dims(1)[1] != st.N || dims(2) != std::vector<int64_t>{st.N} || ot.dims[0] != st.M)
        return bad("shapes must be x [M,K], w [K,N], scale [N] -> [M,N]");
      st.kind = f32 ? kW8A32 : kW8A16;
      st.x = slot_of(op.operands[0]);
      st.w = slot_of(op.operands[1]);
      st.scale = slot_of(op.operands[2]);
      st.out = slot_of(op.result);
    } else if (kind == "i8i8_i32") {
      const bool ints = (elem(0) == "i8" || elem(0) == "ui8") && (elem(1) == "i8" || elem(1) == "ui8");
      st.K = dims(0)[1];
      if (!ints || dims(1)[0] != st.K || dims(1)[1] != st.N || ot.dims[0] != st.M) return bad("expects a [M,K] and b [K,N] of i8 / ui8");
      st.kind = kI8Dot;
      st.x = slot_of(op.operands[0]);
      st.w = slot_of(op.operands[1]);
      st.a_unsigned = elem(0) == "ui8";
      st.b_unsigned = elem(1) == "ui8";
      if (no == 2 && ot.elem == "i32") {
        st.acc_out = slot_of(op.result);
      } else if (no == 4 && ot.elem == "f32" && elem(2) == "f32" && elem(3) == "f32" &&
                 dims(2) == std::vector<int64_t>{st.M} && dims(3) == std::vector<int64_t>{st.N}) {
        st.row = slot_of(op.operands[2]);
        st.col = slot_of(op.operands[3]);
        st.out = slot_of(op.result);
      } else {
        return bad("expects (a, b) -> i32 or (a, b, row: f32 [M], col: f32 [N]) -> f32");
      }
    } else if (kind == "w4a16_g128") {
      st.K = dims(0)[1];
      if (no != 4 || elem(0) != "bf16" || (elem(1) != "ui8" && elem(1) != "i8") || elem(2) != "bf16" || ot.elem != "bf16")
        return bad("expects (x: bf16, wq: ui8, scales: bf16, zeros) -> bf16");
      const bool packed_type = elem(3) == "ui4";
      const bool packed_cfg = cfg.count("zeros_packed") && cfg["zeros_packed"] == "true";
      if (cfg.count("zeros_packed") && cfg["zeros_packed"] != "true" && cfg["zeros_packed"] != "false")
        return bad("\"zeros_packed\" must be true or false");
      st.zeros_packed = packed_type || packed_cfg;
      const int64_t G = st.K / 128;
      const std::vector<int64_t> zshape = (st.zeros_packed && !packed_type) ? std::vector<int64_t>{G, st.N / 2}
                                                                             : std::vector<int64_t>{G, st.N};
      if (st.K % 128 || dims(1)[0] * 2 != st.K || dims(1)[1] != st.N || dims(2) != std::vector<int64_t>{G, st.N} ||
          dims(3) != zshape || ot.dims[0] != st.M || (elem(3) != "ui4" && elem(3) != "ui8" && elem(3) != "i8"))
        return bad("shapes must be x [M,K], wq [K/2,N], scales [K/128,N], zeros [K/128,N] (ui4, or ui8; [K/128,N/2] "
                   "bytes with zeros_packed) -> [M,N]");
      st.kind = kW4A16;
      st.x = slot_of(op.operands[0]);
      st.w = slot_of(op.operands[1]);
      st.scale = slot_of(op.operands[2]);
      st.zeros = slot_of(op.operands[3]);
      st.out = slot_of(op.result);
    } else {
      return set_error(QMM_ERR_INVALID_ARGUMENT,
                       "line %d: backend_config \"op\" must be one of w8a32_perchannel, w8a16_perchannel, i8i8_i32, "
                       "w4a16_g128", op.line);
    }
    st.fused_ops = 1;
    consumed.insert((int)ci);
    static const char* kind_name[] = {"qmm_w8a32_perchannel", "qmm_w8a16_perchannel", "qmm_i8i8_i32", "qmm_w4a16_g128"};
    tracef(plan.trace, "{\"event\":\"custom_call\",\"anchor_line\":%d,\"kernel\":\"%s\",\"M\":%lld,\"N\":%lld,\"K\":%lld}",
           op.line, kind_name[st.kind], (long long)st.M, (long long)st.N, (long long)st.K);
    plan.steps.push_back(st);
  }

  for (size_t di = 0; di < m.ops.size(); ++di) {
    const Op& dot = m.ops[di];
    if (dot.name != "stablehlo.dot_general" && dot.name != "stablehlo.dot") continue;
    Step st;
    std::vector<int> used;
    const std::map<std::string, int> slots_before = plan.slot;
    const size_t temps_before = temp_bytes.size();
    int rc = match(di, st, used);
    std::set<int> mine(used.begin(), used.end());
    if (rc == QMM_OK) {
      // absorbed intermediates must not be used elsewhere
      for (int o : mine) {
        if (m.ops[o].name == "stablehlo.constant") continue;
        const std::string& res = m.ops[o].result;
        const bool is_out = (st.out >= 0 && plan.slot.count(res) && plan.slot[res] == st.out) ||
                            (st.acc_out >= 0 && plan.slot.count(res) && plan.slot[res] == st.acc_out);
        if (is_out) continue;
        bool escapes = result_index(m, res) >= 0;
        for (int u : users[res])
          if (!mine.count(u)) escapes = true;
        if (escapes) {
          rc = set_error(QMM_ERR_UNSUPPORTED, "line %d: %s would be fused into the dot on line %d but its value is "
                         "also used elsewhere", m.ops[o].line, m.ops[o].name.c_str(), dot.line);
          break;
        }
      }
    }
    if (rc == QMM_OK) {
      // an op claimed by an earlier fused step cannot be shared
      for (int o : mine)
        if (consumed.count(o) && m.ops[o].name != "stablehlo.constant")
          rc = set_error(QMM_ERR_UNSUPPORTED, "line %d: %s already belongs to another fused matmul", m.ops[o].line,
                         m.ops[o].name.c_str());
    }
    if (rc == QMM_ERR_UNSUPPORTED) {
      // not fused: forget the slots the attempt created; the dot and its chain run op by op
      plan.slot = slots_before;
      temp_bytes.resize(temps_before);
      char why[512];
      qmm_last_error(why, sizeof(why));
      std::string reason;
      for (const char* c = why; *c; ++c) reason += (*c == '"' || *c == '\\') ? '\'' : *c;
      tracef(plan.trace, "{\"event\":\"not_fused\",\"line\":%d,\"op\":\"%s\",\"reason\":\"%s\"}", dot.line,
             dot.name.c_str(), reason.c_str());
      continue;
    }
    if (rc != QMM_OK) return rc;
    st.fused_ops = (int)mine.size();
    for (int o : mine) consumed.insert(o);
    static const char* kind_name[] = {"qmm_w8a32_perchannel", "qmm_w8a16_perchannel", "qmm_i8i8_i32",
                                      "qmm_w4a16_g128"};
    tracef(plan.trace,
           "{\"event\":\"fused\",\"anchor_line\":%d,\"kernel\":\"%s\",\"M\":%lld,\"N\":%lld,\"K\":%lld,"
           "\"ops_fused\":%d,\"rescale\":%s,\"numerics\":\"%s\"}",
           dot.line, kind_name[st.kind], (long long)st.M, (long long)st.N, (long long)st.K, st.fused_ops,
           (st.kind == kI8Dot && st.out >= 0) ? "true" : "false", st.numerics);
    plan.steps.push_back(st);
  }

  // ---- everything the fused steps did not absorb: one standalone kernel per op
  int fused_count = (int)plan.steps.size();
  for (size_t i = 0; i < m.ops.size(); ++i) {
    if (consumed.count((int)i)) continue;
    const Op& op = m.ops[i];
    // a splat constant that only fused steps looked at needs no buffer
    if (op.name == "stablehlo.constant") {
      bool needed = result_index(m, op.result) >= 0;
      for (int u : users[op.result])
        if (!consumed.count(u)) needed = true;
      if (!needed) continue;
    }
    Step st;
    st.kind = kGeneric;
    st.anchor_line = op.line;
    st.anchor_op = (int)i;
    const TType& ot = op.out_type;
    st.out_dt = dtype_of_elem_early(ot.elem);
    if (st.out_dt < 0)
      return set_error(QMM_ERR_UNSUPPORTED, "line %d: %s produces element type %s, which this backend has no buffers for",
                       op.line, op.name.c_str(), ot.elem.c_str());
    st.count = ot.count();
    for (auto& v : op.operands) {
      if (!type_of(v)) return set_error(QMM_ERR_PARSE, "line %d: %s reads the undefined value %s", op.line, op.name.c_str(), v.c_str());
      st.ins.push_back(slot_of(v));
    }
    st.in_dt = op.in_types.empty() ? st.out_dt : dtype_of_elem_early(op.in_types[0].elem);
    if (st.in_dt < 0)
      return set_error(QMM_ERR_UNSUPPORTED, "line %d: %s reads element type %s, which this backend has no buffers for",
                       op.line, op.name.c_str(), op.in_types[0].elem.c_str());
    st.out = slot_of(op.result);
    const std::string& n = op.name;
    auto need_operands = [&](size_t k) { return op.operands.size() == k && op.in_types.size() >= k; };
    if (n == "stablehlo.convert" && need_operands(1)) {
      st.gop = gConvert;
    } else if ((n == "stablehlo.multiply" || n == "stablehlo.subtract" || n == "stablehlo.add" || n == "stablehlo.and" ||
                n == "stablehlo.shift_right_logical") && need_operands(2)) {
      st.gop = gBinary;
      st.bop = n == "stablehlo.multiply" ? gen::kMul : n == "stablehlo.subtract" ? gen::kSub
               : n == "stablehlo.add" ? gen::kAdd : n == "stablehlo.and" ? gen::kAnd : gen::kShrLogical;
      if (op.in_types[0].count() != st.count || op.in_types[1].count() != st.count)
        return set_error(QMM_ERR_UNSUPPORTED, "line %d: %s with operands of different shapes", op.line, n.c_str());
    } else if (n == "stablehlo.reshape" && need_operands(1)) {
      st.gop = gCopy;  // row-major data does not move
      st.bytes = (size_t)st.count * gen::dtype_bits(st.out_dt) / 8;
    } else if ((n == "stablehlo.broadcast_in_dim" || n == "stablehlo.transpose" || n == "stablehlo.slice") &&
               need_operands(1)) {
      st.gop = gGather;
      const TType& it = op.in_types[0];
      if (it.dims.size() > (size_t)gen::kMaxRank || ot.dims.size() > (size_t)gen::kMaxRank)
        return set_error(QMM_ERR_UNSUPPORTED, "line %d: %s on tensors of rank > %d", op.line, n.c_str(), gen::kMaxRank);
      st.in_dims.assign(it.dims.begin(), it.dims.end());
      st.out_dims.assign(ot.dims.begin(), ot.dims.end());
      st.start.assign(it.dims.size(), 0);
      st.stride.assign(it.dims.size(), 1);
      st.src_of.assign(it.dims.size(), 0);
      if (n == "stablehlo.broadcast_in_dim") {
        std::vector<int64_t> dims = int_list_after(op.body, "dims");
        if (dims.size() != it.dims.size()) return set_error(QMM_ERR_PARSE, "line %d: malformed broadcast_in_dim", op.line);
        for (size_t k = 0; k < dims.size(); ++k) {
          if (dims[k] < 0 || dims[k] >= (int64_t)ot.dims.size() || (it.dims[k] != 1 && it.dims[k] != ot.dims[dims[k]]))
            return set_error(QMM_ERR_PARSE, "line %d: broadcast_in_dim dimensions do not fit", op.line);
          st.src_of[k] = dims[k];
        }
      } else if (n == "stablehlo.transpose") {
        std::vector<int64_t> perm = int_list_after(op.body, "dims");
        if (perm.empty()) perm = int_list_after(op.body, "permutation");
        if (perm.size() != it.dims.size()) return set_error(QMM_ERR_PARSE, "line %d: malformed transpose", op.line);
        for (size_t o = 0; o < perm.size(); ++o) {  // result dimension o is operand dimension perm[o]
          if (perm[o] < 0 || perm[o] >= (int64_t)it.dims.size() || it.dims[perm[o]] != ot.dims[o])
            return set_error(QMM_ERR_PARSE, "line %d: transpose permutation does not fit", op.line);
          st.src_of[perm[o]] = (long long)o;
        }
        // a size-1 operand dimension reads coordinate 0, which is the only one it has
      } else {
        // slice: "[0:4, 2:10:2]" in the pretty form, start_indices / limit_indices / strides otherwise
        std::vector<int64_t> start = int_list_after(op.body, "start_indices"), stride = int_list_after(op.body, "strides");
        if (start.empty()) {
          size_t a = op.body.find('['), b = op.body.find(']');
          if (a == std::string::npos || b == std::string::npos)
            return set_error(QMM_ERR_PARSE, "line %d: malformed slice", op.line);
          for (auto& part : split_top(op.body.substr(a + 1, b - a - 1))) {
            std::vector<long long> f;
            size_t p0 = 0;
            while (true) {
              size_t c = part.find(':', p0);
              f.push_back(atoll(part.substr(p0, c == std::string::npos ? std::string::npos : c - p0).c_str()));
              if (c == std::string::npos) break;
              p0 = c + 1;
            }
            start.push_back(f[0]);
            stride.push_back(f.size() > 2 ? f[2] : 1);
          }
        }
        if (stride.empty()) stride.assign(start.size(), 1);
        if (start.size() != it.dims.size() || stride.size() != it.dims.size() || ot.dims.size() != it.dims.size())
          return set_error(QMM_ERR_PARSE, "line %d: malformed slice", op.line);
        for (size_t k = 0; k < start.size(); ++k) {
          if (start[k] < 0 || stride[k] < 1 || (ot.dims[k] > 0 && start[k] + (ot.dims[k] - 1) * stride[k] >= it.dims[k]))
            return set_error(QMM_ERR_PARSE, "line %d: slice out of range", op.line);
          st.src_of[k] = (long long)k;
          st.start[k] = start[k];
          st.stride[k] = stride[k];
        }
        // the gather kernel reads coordinate 0 of size-1 operand dimensions: give those their start
        for (size_t k = 0; k < start.size(); ++k)
          if (it.dims[k] == 1 && start[k] != 0) return set_error(QMM_ERR_PARSE, "line %d: slice out of range", op.line);
      }
    } else if (n == "stablehlo.concatenate" && !op.operands.empty() && op.in_types.size() == op.operands.size()) {
      st.gop = gConcat;
      size_t p0 = op.body.find("dim");
      size_t e0 = p0 == std::string::npos ? std::string::npos : op.body.find('=', p0);
      if (e0 == std::string::npos) return set_error(QMM_ERR_PARSE, "line %d: concatenate without a dimension", op.line);
      const long long dim = atoll(op.body.c_str() + e0 + 1);
      if (dim < 0 || dim >= (long long)ot.dims.size()) return set_error(QMM_ERR_PARSE, "line %d: bad concatenate dimension", op.line);
      st.outer = st.inner = 1;
      for (long long k = 0; k < dim; ++k) st.outer *= ot.dims[k];
      for (size_t k = dim + 1; k < ot.dims.size(); ++k) st.inner *= ot.dims[k];
      st.out_len = ot.dims[dim];
      long long total = 0;
      for (auto& t : op.in_types) {
        if (t.dims.size() != ot.dims.size()) return set_error(QMM_ERR_PARSE, "line %d: concatenate ranks differ", op.line);
        st.part_len.push_back(t.dims[dim]);
        total += t.dims[dim];
      }
      if (total != st.out_len) return set_error(QMM_ERR_PARSE, "line %d: concatenate sizes do not add up", op.line);
    } else if (n == "stablehlo.constant") {
      st.gop = gFill;
      size_t a = op.body.find("dense<"), b = op.body.rfind('>');
      std::string val = (a == std::string::npos || b == std::string::npos) ? "" : trim(op.body.substr(a + 6, b - a - 6));
      if (val == "true") val = "1";
      if (val == "false") val = "0";
      st.fval = atof(val.c_str());
      st.ival = atoll(val.c_str());
    } else if ((n == "stablehlo.dot_general" || n == "stablehlo.dot") && need_operands(2)) {
      st.gop = gDot;
      const TType &lt = op.in_types[0], &rt = op.in_types[1];
      std::vector<int64_t> lc, rc, lb;
      if (n == "stablehlo.dot_general") {
        size_t e = 0;
        lb = int_list_after(op.body, "batching_dims");
        lc = int_list_after(op.body, "contracting_dims", 0, &e);
        if (!lc.empty()) rc = int_list_after(op.body, "x", e);
        if (lc.empty()) {
          lc = int_list_after(op.body, "lhs_contracting_dimensions");
          rc = int_list_after(op.body, "rhs_contracting_dimensions");
          lb = int_list_after(op.body, "lhs_batching_dimensions");
        }
      } else {
        lc = {(int64_t)lt.dims.size() - 1};
        rc = {0};
      }
      if (!lb.empty() || lc.size() != 1 || rc.size() != 1 || rt.dims.size() != 2 || lt.dims.empty() ||
          lc[0] != (int64_t)lt.dims.size() - 1 || (rc[0] != 0 && rc[0] != 1))
        return set_error(QMM_ERR_UNSUPPORTED,
                         "line %d: %s with these dimension numbers is not supported (need [...,K] x [K,N] or "
                         "[...,K] x [N,K], no batch dimensions)", op.line, n.c_str());
      st.b_transposed = rc[0] == 1;
      st.K = rt.dims[rc[0]];
      st.N = rt.dims[1 - rc[0]];
      st.M = 1;
      for (size_t k = 0; k + 1 < lt.dims.size(); ++k) st.M *= lt.dims[k];
      if (lt.dims.back() != st.K) return set_error(QMM_ERR_PARSE, "line %d: contracting sizes differ", op.line);
      if (dtype_of_elem_early(rt.elem) != st.in_dt)
        return set_error(QMM_ERR_UNSUPPORTED, "line %d: %s with operands of different element types", op.line, n.c_str());
    } else {
      tracef(plan.trace, "{\"event\":\"unsupported\",\"line\":%d,\"op\":\"%s\"}", op.line, n.c_str());
      return set_error(QMM_ERR_UNSUPPORTED,
                       "line %d: %s is not an op this backend executes (fused: int8/int4 dequantisation chains feeding "
                       "dot_general, int8 dot_general; standalone: convert, multiply, subtract, add, and, "
                       "shift_right_logical, broadcast_in_dim, reshape, transpose, slice, concatenate, constant, dot)",
                       op.line, n.c_str());
    }
    if (n != "stablehlo.dot_general" && n != "stablehlo.dot")  // the dot's own line was written with its reason
      tracef(plan.trace, "{\"event\":\"not_fused\",\"line\":%d,\"op\":\"%s\"}", op.line, n.c_str());
    plan.steps.push_back(st);
  }
  if (plan.steps.empty()) return set_error(QMM_ERR_UNSUPPORTED, "the module computes nothing");
  std::stable_sort(plan.steps.begin(), plan.steps.end(),
                   [](const Step& a, const Step& b) { return a.anchor_op < b.anchor_op; });

  // every temporary a step reads must be written by an earlier step
  {
    std::set<int> written;
    for (int a = 0; a < A; ++a) written.insert(a);
    for (const Step& st : plan.steps) {
      std::vector<int> reads = st.ins;
      for (int v : {st.x, st.w, st.scale, st.zeros, st.row, st.col})
        if (v >= 0) reads.push_back(v);
      for (int v : reads)
        if (!written.count(v))
          return set_error(QMM_ERR_UNSUPPORTED, "line %d: a value this step reads is not produced by any executed op",
                           st.anchor_line);
      if (st.out >= 0) written.insert(st.out);
      if (st.acc_out >= 0) written.insert(st.acc_out);
    }
    // results: produced by a step, or a pass-through of an argument / a value returned twice -> copy
    for (int r = 0; r < R; ++r) {
      const std::string& v = m.returns[r];
      const int src = plan.slot.count(v) ? plan.slot[v] : slot_of(v);
      if (src == A + r && written.count(src)) continue;
      if (!written.count(src))
        return set_error(QMM_ERR_UNSUPPORTED, "result %d (%s) is not produced by any executed op", r, v.c_str());
      const TType* t = type_of(v);
      Step cp;
      cp.kind = kGeneric;
      cp.gop = gCopy;
      cp.anchor_op = (int)m.ops.size() + r;
      cp.ins = {src};
      cp.out = A + r;
      cp.bytes = (size_t)t->count() * gen::dtype_bits(dtype_of_elem_early(t->elem)) / 8;
      plan.steps.push_back(cp);
    }
  }

  for (auto& s : plan.steps)
    if (s.kind == kW4A16) {
      size_t w = qmm_w4a16_g128_workspace_bytes(s.M, s.N, s.K);
      const bool prefill = s.M > 32 && s.N >= 128 && s.N % 128 == 0 && s.K >= 128 && s.K % 128 == 0;  // no scratch
      if (w == 0 && !prefill)
        return set_error(QMM_ERR_UNSUPPORTED,
                         "line %d: int4 matmul with M=%lld N=%lld K=%lld is outside the kernels' range (N and K "
                         "must be multiples of 128)",
                         s.anchor_line, (long long)s.M, (long long)s.N, (long long)s.K);
      if (w > plan.scratch) plan.scratch = w;
    }
  plan.scratch = (plan.scratch + 255) / 256 * 256;
  size_t off = plan.scratch;
  for (size_t b : temp_bytes) {
    plan.temp_offset.push_back(off);
    off += b;
  }
  plan.workspace = off;
  tracef(plan.trace, "{\"event\":\"plan\",\"steps\":%d,\"fused\":%d,\"workspace_bytes\":%zu}", (int)plan.steps.size(),
         fused_count, plan.workspace);
  return QMM_OK;
}

}  // namespace hlo
}  // namespace qmm

extern "C" {

struct qmm_plan {
  qmm::hlo::Plan p;
};

int qmm_plan_compile(const char* text, size_t len, qmm_plan** out) {
  using namespace qmm;
  QMM_REQUIRE(text && out, QMM_ERR_INVALID_ARGUMENT, "qmm_plan_compile: null argument");
  *out = nullptr;
  qmm_plan* plan = new qmm_plan();
  if (!hlo::parse_module(text, len, plan->p.mod)) {
    int rc = set_error(QMM_ERR_PARSE, "%s", plan->p.mod.error.c_str());
    delete plan;
    return rc;
  }
  hlo::lift_argument_views(plan->p.mod);
  int rc = hlo::build_plan(plan->p);
  if (getenv("QMM_TRACE_PLAN")) fputs(plan->p.trace.c_str(), stderr);
  if (rc != QMM_OK) {
    delete plan;
    return rc;
  }
  *out = plan;
  return QMM_OK;
}

void qmm_plan_destroy(qmm_plan* plan) {
  if (!plan) return;
  for (auto& kv : plan->p.const_dev) {
    cudaSetDevice(kv.first);
    for (void* p : kv.second) cudaFree(p);
  }
  delete plan;
}

int qmm_plan_num_steps(const qmm_plan* plan) { return plan ? (int)plan->p.steps.size() : 0; }
int qmm_plan_num_args(const qmm_plan* plan) { return plan ? plan->p.mod.num_real_args : 0; }
int qmm_plan_num_fused_steps(const qmm_plan* plan) {
  int n = 0;
  if (plan)
    for (const auto& s : plan->p.steps) n += s.kind != qmm::hlo::kGeneric;
  return n;
}
int qmm_plan_num_results(const qmm_plan* plan) { return plan ? (int)plan->p.mod.returns.size() : 0; }
size_t qmm_plan_workspace_bytes(const qmm_plan* plan) { return plan ? plan->p.workspace : 0; }

static int dtype_of_elem(const std::string& e) {
  if (e == "f32") return QMM_F32;
  if (e == "f16") return QMM_F16;
  if (e == "bf16") return QMM_BF16;
  if (e == "i8" || e == "si8") return QMM_S8;
  if (e == "ui8") return QMM_U8;
  if (e == "i32" || e == "si32") return QMM_S32;
  if (e == "ui4") return QMM_U4;
  if (e == "ui32") return QMM_U32;
  return -1;
}

static int type_info(const qmm::hlo::TType& t, int* dtype, int64_t* dims, int* rank) {
  using namespace qmm;
  const int cap = rank ? *rank : 0;
  QMM_REQUIRE(static_cast<int>(t.dims.size()) <= cap || dims == nullptr, QMM_ERR_INVALID_ARGUMENT,
              "tensor of rank %zu does not fit the caller's %d dimensions", t.dims.size(), cap);
  if (dtype) *dtype = dtype_of_elem(t.elem);
  if (rank) *rank = static_cast<int>(t.dims.size());
  if (dims)
    for (size_t i = 0; i < t.dims.size(); ++i) dims[i] = t.dims[i];
  return QMM_OK;
}

int qmm_plan_arg_info(const qmm_plan* plan, int index, int* dtype, int64_t* dims, int* rank) {
  using namespace qmm;
  QMM_REQUIRE(plan && index >= 0 && index < plan->p.mod.num_real_args, QMM_ERR_INVALID_ARGUMENT,
              "qmm_plan_arg_info: bad plan or index %d", index);
  return type_info(plan->p.mod.arg_types[index], dtype, dims, rank);
}

int qmm_plan_result_info(const qmm_plan* plan, int index, int* dtype, int64_t* dims, int* rank) {
  using namespace qmm;
  QMM_REQUIRE(plan && index >= 0 && index < (int)plan->p.mod.returns.size(), QMM_ERR_INVALID_ARGUMENT,
              "qmm_plan_result_info: bad plan or index %d", index);
  const hlo::Module& m = plan->p.mod;
  const std::string& v = m.returns[index];
  auto d = m.def.find(v);
  if (d != m.def.end()) return type_info(m.ops[d->second].out_type, dtype, dims, rank);
  auto a = m.argi.find(v);
  QMM_REQUIRE(a != m.argi.end(), QMM_ERR_PARSE, "result %d (%s) has no definition", index, v.c_str());
  return type_info(m.arg_types[a->second], dtype, dims, rank);
}

const char* qmm_plan_name(const qmm_plan* plan) { return plan ? plan->p.mod.name.c_str() : ""; }
int qmm_plan_num_replicas(const qmm_plan* plan) { return plan ? plan->p.mod.num_replicas : 0; }
int qmm_plan_num_partitions(const qmm_plan* plan) { return plan ? plan->p.mod.num_partitions : 0; }

double qmm_plan_flops(const qmm_plan* plan) {
  double f = 0;
  if (plan)
    for (const auto& s : plan->p.steps)
      if (s.kind != qmm::hlo::kGeneric || s.gop == qmm::hlo::gDot) f += 2.0 * (double)s.M * (double)s.N * (double)s.K;
  return f;
}

size_t qmm_plan_trace(const qmm_plan* plan, char* buf, size_t cap) {
  if (!plan) return 0;
  const std::string& t = plan->p.trace;
  if (buf && cap) {
    size_t c = t.size() < cap - 1 ? t.size() : cap - 1;
    memcpy(buf, t.data(), c);
    buf[c] = 0;
  }
  return t.size();
}

// Device copies of the lifted constants for the current device (made on the first execution there).
static int constants_on_device(qmm_plan* plan, std::vector<void*>** out) {
  using namespace qmm;
  int dev = 0;
  QMM_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(plan->p.mu);
  auto it = plan->p.const_dev.find(dev);
  if (it == plan->p.const_dev.end()) {
    std::vector<void*> ptrs;
    for (const auto& bytes : plan->p.mod.const_data) {
      void* p = nullptr;
      QMM_CUDA_TRY(cudaMalloc(&p, bytes.empty() ? 256 : bytes.size()));
      if (!bytes.empty()) QMM_CUDA_TRY(cudaMemcpy(p, bytes.data(), bytes.size(), cudaMemcpyHostToDevice));
      ptrs.push_back(p);
    }
    it = plan->p.const_dev.emplace(dev, std::move(ptrs)).first;
  }
  *out = &it->second;
  return QMM_OK;
}

int qmm_plan_execute(const qmm_plan* cplan, const void* const* args, int num_args, void* const* results,
                     int num_results, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace qmm;
  qmm_plan* plan = const_cast<qmm_plan*>(cplan);  // only the cache of constant buffers changes
  QMM_REQUIRE(plan && (args || num_args == 0) && results, QMM_ERR_INVALID_ARGUMENT, "qmm_plan_execute: null argument");
  const hlo::Module& m = plan->p.mod;
  const int A = (int)m.arg_names.size(), R = (int)m.returns.size();
  QMM_REQUIRE(num_args == m.num_real_args && num_results == R, QMM_ERR_INVALID_ARGUMENT,
              "qmm_plan_execute: expected %d arguments and %d results, got %d and %d", m.num_real_args, R, num_args,
              num_results);
  QMM_REQUIRE(plan->p.workspace == 0 || (workspace && workspace_bytes >= plan->p.workspace), QMM_ERR_WORKSPACE,
              "qmm_plan_execute: %zu bytes of workspace required", plan->p.workspace);
  QMM_REQUIRE(plan->p.workspace == 0 || aligned(workspace, 256), QMM_ERR_WORKSPACE,
              "qmm_plan_execute: the workspace must be 256-byte aligned");
  std::vector<void*>* consts = nullptr;
  if (!m.const_data.empty())
    if (int rc = constants_on_device(plan, &consts)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto ptr = [&](int slot) -> void* {
    if (slot < 0) return nullptr;
    if (slot < m.num_real_args) return const_cast<void*>(args[slot]);
    const int first_view = m.num_real_args + (int)m.const_data.size();
    if (slot < first_view) return (*consts)[slot - m.num_real_args];
    if (slot < A) {
      const auto& v = m.views[slot - first_view];
      void* base = v.first < m.num_real_args ? const_cast<void*>(args[v.first]) : (*consts)[v.first - m.num_real_args];
      return static_cast<uint8_t*>(base) + v.second;
    }
    if (slot < A + R) return results[slot - A];
    return static_cast<uint8_t*>(workspace) + plan->p.temp_offset[slot - A - R];
  };
  // Fused steps read arguments and temporaries and write distinct buffers.  A weight-only GEMM step
  // that follows only GEMM steps of this call, none of which produced one of its operands, is
  // launched as independent of them (it fills the SMs their last round leaves idle).  The first
  // step is always ordered behind everything queued before the call.
  bool only_gemms_so_far = true;
  bool first = true;
  std::set<int> written_by_call;
  for (const hlo::Step& s : plan->p.steps) {
    int rc = QMM_OK;
    void* out = ptr(s.out);
    bool independent = !first && only_gemms_so_far;
    for (int v : {s.x, s.w, s.scale})
      if (v >= 0 && written_by_call.count(v)) independent = false;
    first = false;
    if (s.kind != hlo::kW8A16 && s.kind != hlo::kI8Dot) only_gemms_so_far = false;
    if (s.out >= 0) written_by_call.insert(s.out);
    if (s.acc_out >= 0) written_by_call.insert(s.acc_out);
    switch (s.kind) {
      case hlo::kW8A32:
        rc = qmm_w8a32_perchannel((const float*)ptr(s.x), (const int8_t*)ptr(s.w), (const float*)ptr(s.scale),
                                  (float*)out, s.M, s.N, s.K, stream);
        break;
      case hlo::kW8A16: {
        qmm_gemm_ext ext = {};
        ext.struct_size = sizeof(ext);
        ext.flags = independent ? QMM_GEMM_INDEPENDENT : 0u;
        rc = qmm_w8a16_perchannel_ex((const uint16_t*)ptr(s.x), (const int8_t*)ptr(s.w), (const float*)ptr(s.scale),
                                     (uint16_t*)out, s.M, s.N, s.K, s.N, &ext, stream);
        break;
      }
      case hlo::kI8Dot:
        rc = qmm_i8i8_i32(ptr(s.x), ptr(s.w), (int32_t*)ptr(s.acc_out), (const float*)ptr(s.row),
                          (const float*)ptr(s.col), (float*)out, s.M, s.N, s.K, s.a_unsigned, s.b_unsigned, stream);
        break;
      case hlo::kW4A16:
        rc = qmm_w4a16_g128((const uint16_t*)ptr(s.x), (const uint8_t*)ptr(s.w), (const uint16_t*)ptr(s.scale),
                            (const uint8_t*)ptr(s.zeros), s.zeros_packed, (uint16_t*)out, s.M, s.N, s.K, 128,
                            workspace, plan->p.scratch, 0u, stream);
        break;
      case hlo::kGeneric:
        switch (s.gop) {
          case hlo::gConvert: rc = gen::convert(ptr(s.ins[0]), s.in_dt, out, s.out_dt, s.count, st); break;
          case hlo::gBinary: rc = gen::binary(s.bop, ptr(s.ins[0]), ptr(s.ins[1]), out, s.out_dt, s.count, st); break;
          case hlo::gGather:
            rc = gen::gather(ptr(s.ins[0]), out, s.out_dt, s.in_dims.data(), (int)s.in_dims.size(), s.out_dims.data(),
                             (int)s.out_dims.size(), s.src_of.data(), s.start.data(), s.stride.data(), st);
            break;
          case hlo::gConcat: {
            long long off = 0;
            for (size_t k = 0; k < s.ins.size() && rc == QMM_OK; ++k) {
              rc = gen::concat_part(ptr(s.ins[k]), out, s.out_dt, s.outer, s.part_len[k], s.out_len, off, s.inner, st);
              off += s.part_len[k];
            }
            break;
          }
          case hlo::gFill: rc = gen::fill(out, s.out_dt, s.fval, s.ival, s.count, st); break;
          case hlo::gDot:
            rc = gen::dot(ptr(s.ins[0]), ptr(s.ins[1]), out, s.in_dt, s.out_dt, s.M, s.N, s.K, s.b_transposed, st);
            break;
          case hlo::gCopy:
            if (s.bytes && out != ptr(s.ins[0]))
              QMM_CUDA_TRY(cudaMemcpyAsync(out, ptr(s.ins[0]), s.bytes, cudaMemcpyDeviceToDevice, st));
            break;
        }
        break;
    }
    if (rc != QMM_OK) return rc;
  }
  return QMM_OK;
}

}  // extern "C"
