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
// Each match becomes one kernel launch.  Anything left over is a compile error
// that names the op (the reference's convention, api/pjrt_client.cc:211-220):
// there is no fallback executor.  Every decision is recorded as a JSON line
// (`QMM_PLAN_JSON:`), like the reference's JAX_METALLIB_TRACE_PLAN output, so
// tests can assert that a chain was fused.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <set>
#include <string>
#include <vector>

#include "../common.cuh"

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

static bool parse_module(const char* text, size_t len, Module& m) {
  std::string all(text, len);
  std::vector<std::string> lines;
  {
    size_t p = 0;
    while (p <= all.size()) {
      size_t e = all.find('\n', p);
      if (e == std::string::npos) e = all.size();
      lines.push_back(all.substr(p, e - p));
      p = e + 1;
    }
  }
  bool in_main = false, seen_main = false;
  int lineno = 0;
  for (auto& raw : lines) {
    ++lineno;
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
enum StepKind { kW8A32 = 0, kW8A16 = 1, kI8Dot = 2, kW4A16 = 3 };

struct Step {
  StepKind kind;
  int64_t M = 0, N = 0, K = 0;
  int x = -1, w = -1, scale = -1, zeros = -1, row = -1, col = -1;  // argument indices
  int out = -1, acc_out = -1;                                       // result indices (-1 = not returned)
  int a_unsigned = 0, b_unsigned = 0, zeros_packed = 0;
  int anchor_line = 0;
  int fused_ops = 0;
};

struct Plan {
  Module mod;
  std::vector<Step> steps;
  std::string trace;  // JSON lines
  size_t workspace = 0;
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

static int build_plan(Plan& plan) {
  Module& m = plan.mod;
  std::set<int> consumed;  // ops absorbed into a step
  // users of every value, to make sure absorbed intermediates do not escape
  std::map<std::string, std::vector<int>> users;
  for (size_t i = 0; i < m.ops.size(); ++i)
    for (auto& o : m.ops[i].operands) users[o].push_back((int)i);

  for (size_t di = 0; di < m.ops.size(); ++di) {
    const Op& dot = m.ops[di];
    if (dot.name != "stablehlo.dot_general" && dot.name != "stablehlo.dot") continue;
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
    Step st;
    st.M = M; st.N = N; st.K = K;
    st.anchor_line = dot.line;
    std::vector<int> used;
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
      st.acc_out = result_index(m, dot.result);
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
          if (v.dim_of[0] == 0 && v.dim_of[1] == -1 && at.dims[0] == M && got_row < 0) got_row = v.arg;
          else if (v.dim_of[0] == -1 && v.dim_of[1] == 0 && at.dims[0] == N && got_col < 0) got_col = v.arg;
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
        st.out = result_index(m, last);
        for (int o : chain) used.push_back(o);
      }
      if (st.acc_out < 0 && st.out < 0)
        return set_error(QMM_ERR_UNSUPPORTED, "line %d: the integer dot's result is not returned", dot.line);
    } else if (is_float(lt.elem) && lhs_arg != m.argi.end()) {
      st.x = lhs_arg->second;
      // rhs chain
      int ri;
      const Op* r = def_of(m, dot.operands[1], &ri);
      if (!r)
        return set_error(QMM_ERR_UNSUPPORTED,
                         "line %d: dot_general on plain float arguments is not on the quantized-matmul path",
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
        st.w = warg;
        st.scale = sv.arg;
        st.zeros = zv.arg;
        st.zeros_packed = zt.elem == "ui4";  // 4-bit buffers hold two values per byte, low nibble first
        st.out = result_index(m, dot.result);
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
        if (lt.elem == "f32" && ot.elem == "f32") st.kind = kW8A32;
        else if (lt.elem == "bf16" && ot.elem == "bf16") st.kind = kW8A16;
        else
          return set_error(QMM_ERR_UNSUPPORTED, "line %d: %s activations with %s result are not covered",
                           dot.line, lt.elem.c_str(), ot.elem.c_str());
        st.w = warg;
        st.scale = sv.arg;
        st.out = result_index(m, dot.result);
      } else {
        return set_error(QMM_ERR_UNSUPPORTED,
                         "line %d: the rhs of the dot on line %d is produced by %s, which is not a dequantisation "
                         "chain this backend fuses", top->line, dot.line, top->name.c_str());
      }
      if (st.out < 0) {
        auto u = users.find(dot.result);
        if (u != users.end() && !u->second.empty())
          return set_error(QMM_ERR_UNSUPPORTED,
                           "line %d: %s consumes the result of the dot on line %d; ops after the matmul are not "
                           "executed by this backend", m.ops[u->second[0]].line,
                           m.ops[u->second[0]].name.c_str(), dot.line);
        return set_error(QMM_ERR_UNSUPPORTED, "line %d: the dot's result must be a result of @main", dot.line);
      }
    } else {
      return set_error(QMM_ERR_UNSUPPORTED,
                       "line %d: dot_general with %s x %s operands is not on the quantized-matmul path", dot.line,
                       lt.elem.c_str(), rt.elem.c_str());
    }
    // absorbed intermediates must not be used elsewhere
    std::set<int> mine(used.begin(), used.end());
    for (int o : mine) {
      if (m.ops[o].name == "stablehlo.constant") continue;
      const std::string& res = m.ops[o].result;
      bool is_out = (o == (int)di) || result_index(m, res) >= 0;
      for (int u : users[res])
        if (!mine.count(u) && !is_out)
          return set_error(QMM_ERR_UNSUPPORTED,
                           "line %d: %s is fused into the dot on line %d but its value is also used on line %d",
                           m.ops[o].line, m.ops[o].name.c_str(), dot.line, m.ops[u].line);
    }
    st.fused_ops = (int)mine.size();
    for (int o : mine) consumed.insert(o);
    static const char* kind_name[] = {"qmm_w8a32_perchannel", "qmm_w8a16_perchannel", "qmm_i8i8_i32",
                                      "qmm_w4a16_g128"};
    tracef(plan.trace,
           "{\"event\":\"fused\",\"anchor_line\":%d,\"kernel\":\"%s\",\"M\":%lld,\"N\":%lld,\"K\":%lld,"
           "\"ops_fused\":%d,\"rescale\":%s}",
           dot.line, kind_name[st.kind], (long long)M, (long long)N, (long long)K, st.fused_ops,
           (st.kind == kI8Dot && st.out >= 0) ? "true" : "false");
    plan.steps.push_back(st);
  }
  for (size_t i = 0; i < m.ops.size(); ++i) {
    if (consumed.count((int)i)) continue;
    tracef(plan.trace, "{\"event\":\"not_fused\",\"line\":%d,\"op\":\"%s\"}", m.ops[i].line, m.ops[i].name.c_str());
    return set_error(QMM_ERR_UNSUPPORTED,
                     "line %d: %s is not part of a quantized-matmul pattern this backend executes "
                     "(supported: int8/int4 dequantisation chains feeding dot_general, int8 dot_general)",
                     m.ops[i].line, m.ops[i].name.c_str());
  }
  if (plan.steps.empty()) return set_error(QMM_ERR_UNSUPPORTED, "the module contains no dot_general");
  for (auto& s : plan.steps)
    if (s.kind == kW4A16) {
      size_t w = qmm_w4a16_g128_workspace_bytes(s.M, s.N, s.K);
      const bool prefill = s.M > 32 && s.N >= 128 && s.N % 128 == 0 && s.K >= 128 && s.K % 128 == 0;  // no scratch
      if (w == 0 && !prefill)
        return set_error(QMM_ERR_UNSUPPORTED,
                         "line %d: int4 matmul with M=%lld N=%lld K=%lld is outside the kernels' range (N and K "
                         "must be multiples of 128)",
                         s.anchor_line, (long long)s.M, (long long)s.N, (long long)s.K);
      if (w > plan.workspace) plan.workspace = w;
    }
  tracef(plan.trace, "{\"event\":\"plan\",\"steps\":%d,\"workspace_bytes\":%zu}", (int)plan.steps.size(),
         plan.workspace);
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
  int rc = hlo::build_plan(plan->p);
  if (getenv("QMM_TRACE_PLAN")) fputs(plan->p.trace.c_str(), stderr);
  if (rc != QMM_OK) {
    delete plan;
    return rc;
  }
  *out = plan;
  return QMM_OK;
}

void qmm_plan_destroy(qmm_plan* plan) { delete plan; }

int qmm_plan_num_steps(const qmm_plan* plan) { return plan ? (int)plan->p.steps.size() : 0; }
int qmm_plan_num_args(const qmm_plan* plan) { return plan ? (int)plan->p.mod.arg_names.size() : 0; }
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
  QMM_REQUIRE(plan && index >= 0 && index < (int)plan->p.mod.arg_types.size(), QMM_ERR_INVALID_ARGUMENT,
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
    for (const auto& s : plan->p.steps) f += 2.0 * (double)s.M * (double)s.N * (double)s.K;
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

int qmm_plan_execute(const qmm_plan* plan, const void* const* args, int num_args, void* const* results,
                     int num_results, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace qmm;
  QMM_REQUIRE(plan && args && results, QMM_ERR_INVALID_ARGUMENT, "qmm_plan_execute: null argument");
  QMM_REQUIRE(num_args == (int)plan->p.mod.arg_names.size() && num_results == (int)plan->p.mod.returns.size(),
              QMM_ERR_INVALID_ARGUMENT, "qmm_plan_execute: expected %d arguments and %d results, got %d and %d",
              (int)plan->p.mod.arg_names.size(), (int)plan->p.mod.returns.size(), num_args, num_results);
  QMM_REQUIRE(plan->p.workspace == 0 || (workspace && workspace_bytes >= plan->p.workspace), QMM_ERR_WORKSPACE,
              "qmm_plan_execute: %zu bytes of workspace required", plan->p.workspace);
  // Steps read only arguments of @main and write distinct results, so they do not depend on one
  // another: a weight-only GEMM step that follows only GEMM steps of this call is launched as
  // independent of them (it fills the SMs their last round leaves idle).  The first step is always
  // ordered behind everything queued before the call.
  bool only_gemms_so_far = true;
  bool first = true;
  for (const hlo::Step& s : plan->p.steps) {
    int rc = QMM_OK;
    void* out = s.out >= 0 ? results[s.out] : nullptr;
    const bool independent = !first && only_gemms_so_far;
    first = false;
    if (s.kind != hlo::kW8A16 && s.kind != hlo::kI8Dot) only_gemms_so_far = false;
    switch (s.kind) {
      case hlo::kW8A32:
        rc = qmm_w8a32_perchannel((const float*)args[s.x], (const int8_t*)args[s.w], (const float*)args[s.scale],
                                  (float*)out, s.M, s.N, s.K, stream);
        break;
      case hlo::kW8A16:
      {
        qmm_gemm_ext ext = {};
        ext.struct_size = sizeof(ext);
        ext.flags = independent ? QMM_GEMM_INDEPENDENT : 0u;
        rc = qmm_w8a16_perchannel_ex((const uint16_t*)args[s.x], (const int8_t*)args[s.w], (const float*)args[s.scale],
                                     (uint16_t*)out, s.M, s.N, s.K, s.N, &ext, stream);
        break;
      }
      case hlo::kI8Dot:
        rc = qmm_i8i8_i32(args[s.x], args[s.w], s.acc_out >= 0 ? (int32_t*)results[s.acc_out] : nullptr,
                          s.row >= 0 ? (const float*)args[s.row] : nullptr,
                          s.col >= 0 ? (const float*)args[s.col] : nullptr, (float*)out, s.M, s.N, s.K,
                          s.a_unsigned, s.b_unsigned, stream);
        break;
      case hlo::kW4A16:
        rc = qmm_w4a16_g128((const uint16_t*)args[s.x], (const uint8_t*)args[s.w], (const uint16_t*)args[s.scale],
                            (const uint8_t*)args[s.zeros], s.zeros_packed, (uint16_t*)out, s.M, s.N, s.K, 128,
                            workspace, workspace_bytes, 0u, stream);
        break;
    }
    if (rc != QMM_OK) return rc;
  }
  return QMM_OK;
}

}  // extern "C"
