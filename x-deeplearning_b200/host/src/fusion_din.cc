// Graph-fusion patterns that turn the op-by-op DIN graph back into the fused operators.
//
// The reference expresses a fusion as an ordered list of pattern nodes plus a rewrite
// (blaze/blaze/graph/pattern/in_order_pattern.h:18-57) and applies all registered patterns until nothing
// changes (blaze/blaze/graph/fusion_pattern.cc:187-217). The same shape here: a Pattern is a list of nodes
// (operator type + symbolic input names); matching unifies the symbols with blob names of the NetDef, a
// match is accepted only when every blob it would remove is consumed inside the match, and the rewrite
// replaces the matched operators by one. Two patterns cover rows 7-29 of the shipped DIN graph
// (blaze/tools/example_model/din/model/graph_ulf.txt):
//   attention  Sub, Mul, BroadcastTo x2, Concat, Gemm (+act) x2, Gemm, Reshape, MatMul, Reshape -> DinAttention
//   tower      ReduceSum, Mul, Sub, BroadcastTo, Concat, Fuse, Gemm + Dice x2, Gemm, Softmax   -> DinTower
// Both need an fp16 model (the fused kernels are fp16 tensor-core kernels); an fp32 graph is left as it is.
#include <algorithm>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "runtime.h"

namespace blaze {
namespace {

struct PatternNode {
  std::string out;                    // symbol of the node's single output
  std::string type;
  std::vector<std::string> in;        // symbols; every one must bind
  bool commutative = false;           // the first two inputs may come in either order
};

struct Match {
  std::map<std::string, std::string> sym;   // symbol -> blob name
  std::vector<int> ops;                     // matched operator indices, pattern order
};

class Matcher {
 public:
  Matcher(const NetDef& def, const std::vector<PatternNode>& pat) : def_(def), pat_(pat) {}

  // every match whose first pattern node is operator `first`
  bool MatchFrom(int first, Match* m) {
    m->sym.clear();
    m->ops.assign(pat_.size(), -1);
    return Extend(0, first, m);
  }

 private:
  bool Bind(Match* m, const std::string& s, const std::string& blob, std::vector<std::string>* undo) {
    auto it = m->sym.find(s);
    if (it != m->sym.end()) return it->second == blob;
    m->sym[s] = blob;
    undo->push_back(s);
    return true;
  }

  bool TryOp(size_t pi, int oi, bool swapped, Match* m) {
    const PatternNode& p = pat_[pi];
    const OperatorDef& op = def_.op[oi];
    if (op.type != p.type || op.output.size() != 1 || op.input.size() != p.in.size()) return false;
    for (int used : m->ops)
      if (used == oi) return false;
    std::vector<std::string> undo;
    bool ok = Bind(m, p.out, op.output[0], &undo);
    for (size_t k = 0; ok && k < p.in.size(); ++k) {
      size_t src = k;
      if (swapped && k < 2) src = 1 - k;
      ok = Bind(m, p.in[k], op.input[src], &undo);
    }
    if (ok) {
      m->ops[pi] = oi;
      if (pi + 1 == pat_.size() || Extend(pi + 1, -1, m)) return true;
      m->ops[pi] = -1;
    }
    for (const auto& s : undo) m->sym.erase(s);
    return false;
  }

  bool Extend(size_t pi, int forced, Match* m) {
    for (int oi = forced >= 0 ? forced : 0; oi < (int)def_.op.size(); ++oi) {
      if (TryOp(pi, oi, false, m)) return true;
      if (pat_[pi].commutative && TryOp(pi, oi, true, m)) return true;
      if (forced >= 0) break;
    }
    return false;
  }

  const NetDef& def_;
  const std::vector<PatternNode>& pat_;
};

struct GraphView {
  std::map<std::string, std::vector<int>> consumers;
  std::map<std::string, int> producer;
  std::set<std::string> ext_out;
  explicit GraphView(const NetDef& def) {
    for (size_t i = 0; i < def.op.size(); ++i) {
      for (const auto& in : def.op[i].input) consumers[in].push_back((int)i);
      for (const auto& out : def.op[i].output) producer[out] = (int)i;
    }
    for (const auto& v : def.external_output) ext_out.insert(v.name);
  }
};

// true when every blob named by `internal` symbols is produced and consumed inside the match only
bool Closed(const NetDef& def, const GraphView& gv, const Match& m, const std::vector<std::string>& internal) {
  std::set<int> inside(m.ops.begin(), m.ops.end());
  for (const auto& s : internal) {
    const std::string& blob = m.sym.at(s);
    if (gv.ext_out.count(blob)) return false;
    auto it = gv.consumers.find(blob);
    if (it == gv.consumers.end()) continue;
    for (int c : it->second)
      if (!inside.count(c)) return false;
  }
  (void)def;
  return true;
}

const OperatorDef* ConstantOf(const NetDef& def, const GraphView& gv, const std::string& blob) {
  auto it = gv.producer.find(blob);
  if (it == gv.producer.end() || def.op[it->second].type != "ConstantFill") return nullptr;
  return &def.op[it->second];
}

int ConstantDtype(const OperatorDef* c) {
  if (!c) return -1;
  const Argument* dt = c->FindArg("dtype");
  return dt && dt->has_i ? (int)dt->i : kFloat;
}

std::vector<int64_t> ConstantInts(const OperatorDef* c) {
  std::vector<int64_t> v;
  if (!c) return v;
  if (const Argument* a = c->FindArg("value")) {
    v = a->ints;
    if (v.empty()) v.assign(a->floats.begin(), a->floats.end());
  }
  return v;
}

int64_t IntArg(const OperatorDef& op, const char* name, int64_t dflt) {
  const Argument* a = op.FindArg(name);
  return a ? (a->has_i ? a->i : (int64_t)a->f) : dflt;
}

bool PlainGemm(const OperatorDef& g) {
  auto flag = [&](const char* n) { return IntArg(g, n, 0) != 0; };
  auto scalar = [&](const char* n) {
    const Argument* a = g.FindArg(n);
    return a ? (a->has_f ? a->f : (a->has_i ? (float)a->i : 1.f)) : 1.f;
  };
  return !flag("transA") && !flag("transB") && scalar("alpha") == 1.f && scalar("beta") == 1.f && !g.FindArg("epilogue");
}

// removes the matched operators and puts `fused` where the last of them was
void Replace(NetDef* def, const Match& m, const OperatorDef& fused) {
  std::vector<int> idx = m.ops;
  std::sort(idx.begin(), idx.end());
  const int at = idx.back();
  def->op[at] = fused;
  for (size_t k = idx.size() - 1; k-- > 0;) def->op.erase(def->op.begin() + idx[k]);
}

// activation between two Gemm nodes of the attention MLP: 0 none, 1 Sigmoid, 2 Dice
void ActNodes(std::vector<PatternNode>* pat, int act, const std::string& h, const std::string& y, const std::string& tag) {
  if (act == XB_ACT_DICE) pat->push_back({y, "Dice", {h, "g" + tag, "m" + tag, "v" + tag}});
  else if (act == XB_ACT_SIGMOID) pat->push_back({y, "Sigmoid", {h}});
}

bool FuseAttentionOnce(NetDef* def, int act) {
  std::vector<PatternNode> pat;
  pat.push_back({"x", "Concat", {"bq", "bk", "sub", "mul"}});
  pat.push_back({"sub", "Sub", {"q", "k"}});
  pat.push_back({"mul", "Mul", {"q", "k"}, true});
  pat.push_back({"bq", "BroadcastTo", {"q", "sub"}});
  pat.push_back({"bk", "BroadcastTo", {"k", "sub"}});
  pat.push_back({"h0", "Gemm", {"x", "W0", "b0"}});
  const std::string y0 = act == XB_ACT_NONE ? "h0" : "y0", y1 = act == XB_ACT_NONE ? "h1" : "y1";
  ActNodes(&pat, act, "h0", "y0", "0");
  pat.push_back({"h1", "Gemm", {y0, "W1", "b1"}});
  ActNodes(&pat, act, "h1", "y1", "1");
  pat.push_back({"s", "Gemm", {y1, "W2", "b2"}});
  pat.push_back({"w", "Reshape", {"s", "wshape"}});
  pat.push_back({"a3", "MatMul", {"w", "k"}});
  pat.push_back({"att", "Reshape", {"a3", "ashape"}});
  std::vector<std::string> internal = {"x", "sub", "mul", "bq", "bk", "h0", "h1", "s", "w", "a3"};
  if (act != XB_ACT_NONE) { internal.push_back("y0"); internal.push_back("y1"); }

  const GraphView gv(*def);
  Matcher matcher(*def, pat);
  for (int i = 0; i < (int)def->op.size(); ++i) {
    if (def->op[i].type != "Concat" || def->op[i].input.size() != 4) continue;
    Match m;
    if (!matcher.MatchFrom(i, &m) || !Closed(*def, gv, m, internal)) continue;
    auto op_of = [&](const char* sym) -> const OperatorDef& { return def->op[gv.producer.at(m.sym.at(sym))]; };
    // the concat is over the feature axis of [n, T, d] tensors, the Gemm layers are plain, the weights are
    // fp16 constants, the score is reshaped to [n, 1, T] and the result to [n, d]
    if (IntArg(op_of("x"), "axis", 1) != 2) continue;
    if (!PlainGemm(op_of("h0")) || !PlainGemm(op_of("h1")) || !PlainGemm(op_of("s"))) continue;
    bool consts = true;
    std::vector<std::string> weights = {"W0", "b0", "W1", "b1", "W2", "b2"};
    if (act == XB_ACT_DICE) for (const char* s : {"g0", "m0", "v0", "g1", "m1", "v1"}) weights.push_back(s);
    for (const auto& s : weights) consts = consts && ConstantDtype(ConstantOf(*def, gv, m.sym.at(s))) == kFloat16;
    if (!consts) continue;
    const std::vector<int64_t> ws = ConstantInts(ConstantOf(*def, gv, m.sym.at("wshape")));
    const std::vector<int64_t> as = ConstantInts(ConstantOf(*def, gv, m.sym.at("ashape")));
    if (ws.size() != 3 || ws[1] != 1 || as.size() != 2) continue;
    if (IntArg(op_of("a3"), "transA", 0) || IntArg(op_of("a3"), "transB", 0)) continue;

    OperatorDef fused;
    fused.type = "DinAttention";
    fused.name = m.sym.at("att");
    fused.has_device_option = def->op[i].has_device_option;
    fused.device_option = def->op[i].device_option;
    fused.input = {m.sym.at("q"), m.sym.at("k")};
    for (const auto& s : weights) fused.input.push_back(m.sym.at(s));
    fused.output = {m.sym.at("att")};
    Argument a;
    a.name = "act"; a.has_i = true; a.i = act;
    fused.arg.push_back(a);
    Replace(def, m, fused);
    return true;
  }
  return false;
}

bool FuseTowerOnce(NetDef* def) {
  std::vector<PatternNode> pat;
  pat.push_back({"x", "Fuse", {"user", "cs"}});
  pat.push_back({"cs", "Concat", {"q", "hb", "mq", "att", "sq"}});
  pat.push_back({"hb", "BroadcastTo", {"hs", "q"}});
  pat.push_back({"mq", "Mul", {"q", "hs"}, true});
  pat.push_back({"sq", "Sub", {"q", "hs"}});
  pat.push_back({"hs", "ReduceSum", {"k"}});
  pat.push_back({"h1", "Gemm", {"x", "W1", "b1"}});
  pat.push_back({"y1", "Dice", {"h1", "g1", "m1", "v1"}});
  pat.push_back({"h2", "Gemm", {"y1", "W2", "b2"}});
  pat.push_back({"y2", "Dice", {"h2", "g2", "m2", "v2"}});
  pat.push_back({"lg", "Gemm", {"y2", "W3", "b3"}});
  pat.push_back({"out", "Softmax", {"lg"}});
  const std::vector<std::string> internal = {"x", "cs", "hb", "mq", "sq", "hs", "h1", "y1", "h2", "y2", "lg"};
  const std::vector<std::string> weights = {"W1", "b1", "g1", "m1", "v1", "W2", "b2", "g2", "m2", "v2", "W3", "b3"};

  const GraphView gv(*def);
  Matcher matcher(*def, pat);
  for (int i = 0; i < (int)def->op.size(); ++i) {
    if (def->op[i].type != "Fuse") continue;
    Match m;
    if (!matcher.MatchFrom(i, &m) || !Closed(*def, gv, m, internal)) continue;
    auto op_of = [&](const char* sym) -> const OperatorDef& { return def->op[gv.producer.at(m.sym.at(sym))]; };
    if (IntArg(op_of("cs"), "axis", 1) != 1 || IntArg(op_of("out"), "axis", 1) != 1) continue;
    if (IntArg(op_of("hs"), "axis", 0) != 1 || IntArg(op_of("hs"), "keepdims", 1) != 0) continue;
    if (!PlainGemm(op_of("h1")) || !PlainGemm(op_of("h2")) || !PlainGemm(op_of("lg"))) continue;
    if (IntArg(op_of("y1"), "nosqrt", 0) || IntArg(op_of("y2"), "nosqrt", 0)) continue;
    bool consts = true;
    for (const auto& s : weights) consts = consts && ConstantDtype(ConstantOf(*def, gv, m.sym.at(s))) == kFloat16;
    if (!consts) continue;
    // `att` must come from the fused attention unit: DinTower reads q, k and att in its layouts
    auto pa = gv.producer.find(m.sym.at("att"));
    if (pa == gv.producer.end() || def->op[pa->second].type != "DinAttention") continue;
    if (def->op[pa->second].input[1] != m.sym.at("k")) continue;

    OperatorDef fused;
    fused.type = "DinTower";
    fused.name = m.sym.at("out");
    fused.has_device_option = def->op[i].has_device_option;
    fused.device_option = def->op[i].device_option;
    fused.input = {m.sym.at("user"), m.sym.at("q"), m.sym.at("k"), m.sym.at("att")};
    for (const auto& s : weights) fused.input.push_back(m.sym.at(s));
    fused.output = {m.sym.at("out")};
    const std::string out = m.sym.at("out");
    Replace(def, m, fused);
    // the fused tower writes fp32 probabilities
    for (auto& v : def->external_output)
      if (v.name == out) v.dtype = kFloat;
    return true;
  }
  return false;
}

// constants (weights re-packed elsewhere, reshape targets) that nothing reads any more
void DropDeadConstants(NetDef* def) {
  std::map<std::string, int> consumers;
  for (const auto& op : def->op)
    for (const auto& in : op.input) ++consumers[in];
  std::set<std::string> ext_out;
  for (const auto& v : def->external_output) ext_out.insert(v.name);
  for (size_t i = def->op.size(); i-- > 0;) {
    const OperatorDef& op = def->op[i];
    if (op.type == "ConstantFill" && op.output.size() == 1 && consumers[op.output[0]] == 0 && !ext_out.count(op.output[0]))
      def->op.erase(def->op.begin() + i);
  }
}

}  // namespace

int FuseDinSubgraphs(NetDef* def) {
  int fused = 0;
  bool changed = true;
  while (changed) {                       // to a fixed point, as the reference's pattern driver does
    changed = false;
    for (int act : {XB_ACT_DICE, XB_ACT_SIGMOID, XB_ACT_NONE})
      while (FuseAttentionOnce(def, act)) { changed = true; ++fused; }
    while (FuseTowerOnce(def)) { changed = true; ++fused; }
  }
  if (fused) DropDeadConstants(def);
  return fused;
}

}  // namespace blaze
