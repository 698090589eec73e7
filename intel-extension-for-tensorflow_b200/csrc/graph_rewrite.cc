// Graph-side routing of the quantized ops, free of TensorFlow types: which stock-TensorFlow INT8 node becomes which
// `_ITEX*` node, under which condition, and which attrs the new node gets besides a copy of the old ones.
//
// This is what the reference's layout pass does for these ops (the rename table of
// itex/core/graph/native_layout/native_layout.cc:113-199; the predicates RewriteQuantize and RewriteQuantizeReshape,
// itex/core/graph/utils/layout_utils.cc:315-354,392-400; the attr copiers CopyAttrsQuantizedConv2D / CopyAttrsQuantizedMatMul /
// CopyAttrsQuantize, layout_utils.cc:471-542), restricted to the ops this library implements.  A TF_InitGraph
// optimizer calls itexb_rewrite_node for every node and, when it answers with a new op name, replaces the node by one
// of that name with the old node's attrs plus the returned ones - after which the graph dispatches to the kernels of
// the op layer exactly as a graph the reference rewrote does.
#include <cstring>
#include <string>

#include "op_kernel.h"

namespace itexb {
namespace {

enum CopyKind { kCopyAll, kCopyConv2D, kCopyMatMul, kCopyQuantize };
enum Predicate { kAlways, kQuantizeRule, kReshapeRule };

struct Rule {
  const char* from;
  const char* to;
  CopyKind copy;
  Predicate when;
};

// Entries of the reference's table whose target op this library registers.
const Rule kRules[] = {
    {"Dequantize", "_ITEXDequantize", kCopyAll, kQuantizeRule},
    {"QuantizeV2", "_ITEXQuantizeV2", kCopyQuantize, kQuantizeRule},
    {"QuantizedAvgPool", "ITEXQuantizedAvgPool", kCopyAll, kAlways},
    {"QuantizedMaxPool", "_ITEXQuantizedMaxPool", kCopyAll, kAlways},
    {"QuantizedReshape", "_ITEXQuantizedReshape", kCopyAll, kReshapeRule},
    {"QuantizedConv2D", "_ITEXQuantizedConv2D", kCopyConv2D, kAlways},
    {"QuantizedConv2DAndRequantize", "_ITEXQuantizedConv2DAndRequantize", kCopyConv2D, kAlways},
    {"QuantizedConv2DPerChannel", "_ITEXQuantizedConv2DPerChannel", kCopyConv2D, kAlways},
    {"QuantizedConv2DWithBias", "_ITEXQuantizedConv2DWithBias", kCopyConv2D, kAlways},
    {"QuantizedConv2DWithBiasAndRelu", "_ITEXQuantizedConv2DWithBiasAndRelu", kCopyConv2D, kAlways},
    {"QuantizedConv2DWithBiasAndReluAndRequantize", "_ITEXQuantizedConv2DWithBiasAndReluAndRequantize", kCopyConv2D, kAlways},
    {"QuantizedConv2DWithBiasAndRequantize", "_ITEXQuantizedConv2DWithBiasAndRequantize", kCopyConv2D, kAlways},
    {"QuantizedConv2DWithBiasSignedSumAndReluAndRequantize", "_ITEXQuantizedConv2DWithBiasSignedSumAndReluAndRequantize", kCopyConv2D,
     kAlways},
    {"QuantizedConv2DWithBiasSumAndReluAndRequantize", "_ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize", kCopyConv2D, kAlways},
    {"QuantizedMatMulWithBias", "_ITEXQuantizedMatMulWithBias", kCopyMatMul, kAlways},
    {"QuantizedMatMulWithBiasAndDequantize", "_ITEXQuantizedMatMulWithBiasAndDequantize", kCopyMatMul, kAlways},
    {"QuantizedMatMulWithBiasAndRelu", "_ITEXQuantizedMatMulWithBiasAndRelu", kCopyMatMul, kAlways},
    {"QuantizedMatMulWithBiasAndReluAndRequantize", "_ITEXQuantizedMatMulWithBiasAndReluAndRequantize", kCopyMatMul, kAlways},
    {"QuantizedMatMulWithBiasAndRequantize", "_ITEXQuantizedMatMulWithBiasAndRequantize", kCopyMatMul, kAlways},
    {"_QuantizedBatchMatMul", "_ITEXQuantizedBatchMatMul", kCopyAll, kAlways},
    {"_QuantizedBatchMatMulV2AndDequantize", "_ITEXQuantizedBatchMatMulV2AndDequantize", kCopyAll, kAlways},
    {"_QuantizedFusedBatchMatMulV2AndDequantize", "_ITEXQuantizedFusedBatchMatMulV2AndDequantize", kCopyAll, kAlways},
    {"_QuantizedConv2D", "_ITEXQuantizedConv2DV2", kCopyAll, kAlways},
    {"_QuantizedFusedMatMul", "_ITEXQuantizedFusedMatMul", kCopyMatMul, kAlways},
    {"_QuantizedFusedMatMulAndDequantize", "_ITEXQuantizedFusedMatMulAndDequantize", kCopyMatMul, kAlways},
    {"_QuantizedFusedMatMulAndRequantize", "_ITEXQuantizedFusedMatMulAndRequantize", kCopyMatMul, kAlways},
    {"_QuantizedMatMul", "_ITEXQuantizedMatMul", kCopyAll, kAlways},
    {"_QuantizedTranspose", "_ITEXQuantizedTranspose", kCopyAll, kAlways},
};

// RewriteQuantize: MIN_COMBINED is never rewritten; a MIN_FIRST Dequantize stays on the stock kernel when the node is
// placed on the GPU; SCALED quantization is only taken over with HALF_TO_EVEN rounding (Dequantize has no round_mode).
bool QuantizeRule(const std::string& op, const AttrMap& attrs, bool on_gpu, int* status) {
  std::string mode;
  *status = attrs.GetString("mode", &mode);
  if (*status != ITEXB_OK) return false;
  if (mode == "MIN_COMBINED") return false;
  if (mode == "MIN_FIRST" && op == "Dequantize" && on_gpu) return false;
  std::string round_mode;
  if (attrs.Has("round_mode")) {
    *status = attrs.GetString("round_mode", &round_mode);
    if (*status != ITEXB_OK) return false;
    if (mode == "SCALED" && round_mode != "HALF_TO_EVEN") return false;
  }
  return true;
}

void AddString(itexb_rewrite_result_t* r, const char* name, const char* value) {
  itexb_attr_t& a = r->added[r->num_added++];
  std::memset(&a, 0, sizeof(a));
  a.name = name;
  a.type = ITEXB_ATTR_STRING;
  a.s = value;
}
void AddScalar(itexb_rewrite_result_t* r, const char* name, int type, int64_t value) {
  itexb_attr_t& a = r->added[r->num_added++];
  std::memset(&a, 0, sizeof(a));
  a.name = name;
  a.type = type;
  a.i = value;
}

}  // namespace
}  // namespace itexb

using namespace itexb;

extern "C" int itexb_rewrite_node(const itexb_rewrite_query_t* q, itexb_rewrite_result_t* r) {
  ITEXB_REQUIRE(q != nullptr && r != nullptr && q->op != nullptr, ITEXB_INVALID_ARGUMENT, "rewrite_node: NULL argument");
  std::memset(r, 0, sizeof(*r));
  const std::string op(q->op);
  const Rule* rule = nullptr;
  for (const Rule& x : kRules)
    if (op == x.from) rule = &x;
  if (rule == nullptr) return ITEXB_OK;  // not an op of this path: left alone
  AttrMap attrs(q->attrs, q->attrs == nullptr ? 0 : q->num_attrs);
  if (rule->when == kQuantizeRule) {
    int st = ITEXB_OK;
    const bool yes = QuantizeRule(op, attrs, q->on_gpu != 0, &st);
    if (st != ITEXB_OK) return st;  // a Quantize / Dequantize node without `mode` is malformed (the reference CHECK-fails)
    if (!yes) return ITEXB_OK;
  }
  if (rule->when == kReshapeRule) {
    // RewriteQuantizeReshape: only a qint8 reshape is taken over
    int t = 0;
    ITEXB_RETURN_IF_ERROR(attrs.GetType("T", &t));
    if (t != ITEXB_DT_QINT8) return ITEXB_OK;
  }
  switch (rule->copy) {
    case kCopyAll: break;
    case kCopyConv2D: {
      // out_type must be there (CHECK in the reference); data_format is fixed to NHWC; Tbias, when the node has it, is
      // carried over explicitly
      int out_type = 0;
      ITEXB_RETURN_IF_ERROR(attrs.GetType("out_type", &out_type));
      AddString(r, "data_format", "NHWC");
      int tbias = 0;
      if (attrs.Has("Tbias")) {
        ITEXB_RETURN_IF_ERROR(attrs.GetType("Tbias", &tbias));
        AddScalar(r, "Tbias", ITEXB_ATTR_TYPE, tbias);
      }
      break;
    }
    case kCopyMatMul: {
      int toutput = 0, tbias = 0;
      ITEXB_RETURN_IF_ERROR(attrs.GetType("Toutput", &toutput));
      if (attrs.Has("Tbias")) {
        ITEXB_RETURN_IF_ERROR(attrs.GetType("Tbias", &tbias));
        AddScalar(r, "Tbias", ITEXB_ATTR_TYPE, tbias);
      }
      break;
    }
    case kCopyQuantize:
      // QuantizeV2 has no `dtype` attr: the new op's input type defaults to float; the classic asymmetric algorithm is
      // chosen when every consumer of the quantized output is a Dequantize (a graph quantized for oneDNN Graph)
      if (!attrs.Has("dtype")) AddScalar(r, "dtype", ITEXB_ATTR_TYPE, ITEXB_DT_FLOAT);
      AddScalar(r, "classic_asymmetric_algorithm", ITEXB_ATTR_BOOL, q->all_consumers_are_dequantize != 0 ? 1 : 0);
      break;
  }
  r->new_op = rule->to;
  return ITEXB_OK;
}

extern "C" int itexb_rewrite_rule(int index, const char** from, const char** to) {
  const int n = int(sizeof(kRules) / sizeof(kRules[0]));
  if (index < 0 || index >= n) return ITEXB_NOT_FOUND;
  if (from != nullptr) *from = kRules[index].from;
  if (to != nullptr) *to = kRules[index].to;
  return ITEXB_OK;
}
