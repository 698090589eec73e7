// Op definitions of the ops this library implements under names TensorFlow does not define itself: the input, output
// and attr specification strings a plugin hands to TF_OpDefinitionBuilderAddInput / AddOutput / AddAttr before
// TF_RegisterOpDefinition, as the reference registers them (itex/core/ops/nn_ops.cc:738-4760 for the quantized ops,
// itex/core/ops/fp8_ops.cc:22-226 for the FP8 ops; registration pattern at nn_ops.cc:1070-1102).  The strings are the
// interface: a graph rewritten by the reference's passes carries exactly these argument and attr names, so a drop-in
// replacement registers them verbatim.  tests/golden/op_defs.json holds the same data extracted mechanically from the
// reference (tests/golden/make_opdef_fixture.py); tests/test_abi.py compares the two.
#include <cstring>
#include <string>

#include "common.h"

namespace itexb {
namespace {

struct OpDefEntry {
  const char* name;
  const char* const* inputs;
  int num_inputs;
  const char* const* outputs;
  int num_outputs;
  const char* const* attrs;
  int num_attrs;
};

const char* const k0_inputs[] = {
    "x: int8",
    "x_scale_inv: float"};
const char* const k0_outputs[] = {
    "y: out_dtype"};
const char* const k0_attrs[] = {
    "out_dtype: {float, bfloat16, half}",
    "fp8_meta_index: int",
    "fp8_dtype: {'E4M3', 'E5M2'}"};
const char* const k1_inputs[] = {
    "inp: in_dtype",
    "amax: float",
    "scale: float"};
const char* const k1_outputs[] = {
    "gelu_out: int8"};
const char* const k1_attrs[] = {
    "fp8_meta_index: int",
    "in_dtype: {float, bfloat16, half, int8}",
    "fp8_dtype: {'E4M3', 'E5M2'}"};
const char* const k2_inputs[] = {
    "x: in_dtype",
    "gamma: weight_dtype",
    "beta: weight_dtype",
    "z_amax: float",
    "z_scale: float"};
const char* const k2_outputs[] = {
    "z: out_dtype",
    "mu: float",
    "rsigma: float"};
const char* const k2_attrs[] = {
    "fp8_meta_index: int",
    "in_dtype: {float, bfloat16, half, int8}",
    "weight_dtype: {float, bfloat16, half}",
    "out_dtype: {float, bfloat16, half, int8}",
    "epsilon: float = 0.0001",
    "fp8_dtype: {'E4M3', 'E5M2'}"};
const char* const k3_inputs[] = {
    "src: int8",
    "weight: int8",
    "bias: sum_dtype",
    "post_add: sum_dtype",
    "a_scale_inv: float",
    "b_scale_inv: float",
    "c_amax: float",
    "c_scale: float"};
const char* const k3_outputs[] = {
    "dst: out_dtype"};
const char* const k3_attrs[] = {
    "fp8_meta_index_a: int",
    "fp8_meta_index_b: int",
    "fp8_meta_index_c: int = -1",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "use_bias: bool = false",
    "has_post_add: bool = false",
    "sum_dtype: {float, bfloat16, half}",
    "out_dtype: {float, bfloat16, half, int8}",
    "fp8_dtype_a: {'E4M3', 'E5M2'}",
    "fp8_dtype_b: {'E4M3', 'E5M2'}",
    "fp8_dtype_c: {'E4M3', 'E5M2', ''} = ''"};
const char* const k4_inputs[] = {
    "x: in_dtype",
    "x_amax: float",
    "x_scale: float"};
const char* const k4_outputs[] = {
    "y: int8"};
const char* const k4_attrs[] = {
    "in_dtype: {float, bfloat16, half}",
    "fp8_meta_index: int",
    "fp8_dtype: {'E4M3', 'E5M2'}"};
const char* const k5_inputs[] = {
    "grad: grad_dtype",
    "amax: float",
    "scale: float"};
const char* const k5_outputs[] = {
    "quantize_out: int8",
    "dbias: grad_dtype"};
const char* const k5_attrs[] = {
    "fp8_meta_index: int",
    "grad_dtype: {float, bfloat16, half, int8}",
    "fp8_dtype: {'E4M3', 'E5M2'}"};
const char* const k6_inputs[] = {
    "grad: grad_dtype",
    "gelu_inp: in_dtype",
    "amax: float",
    "scale: float"};
const char* const k6_outputs[] = {
    "dgelu: int8",
    "dbias: grad_dtype"};
const char* const k6_attrs[] = {
    "fp8_meta_index: int",
    "in_dtype: {float, bfloat16, half, int8}",
    "grad_dtype: {float, bfloat16, half, int8}",
    "fp8_dtype: {'E4M3', 'E5M2'}"};
const char* const k7_inputs[] = {
    "input: T",
    "min_input: float",
    "max_input: float"};
const char* const k7_outputs[] = {
    "output: T",
    "min_output: float",
    "max_output: float"};
const char* const k7_attrs[] = {
    "T: quantizedtype",
    "ksize: list(int) >= 4",
    "strides: list(int) >= 4"};
const char* const k8_inputs[] = {
    "input: T",
    "min_range: float",
    "max_range: float"};
const char* const k8_outputs[] = {
    "output: dtype"};
const char* const k8_attrs[] = {
    "T: quantizedtype",
    "mode: {'MIN_COMBINED', 'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "narrow_range: bool = false",
    "axis: int = -1",
    "dtype: {bfloat16, float} = DT_FLOAT"};
const char* const k9_inputs[] = {
    "input: dtype",
    "min_range: float",
    "max_range: float"};
const char* const k9_outputs[] = {
    "output: T",
    "output_min: float",
    "output_max: float"};
const char* const k9_attrs[] = {
    "T: quantizedtype",
    "mode: {'MIN_COMBINED', 'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "round_mode: {'HALF_AWAY_FROM_ZERO', 'HALF_TO_EVEN'} = 'HALF_AWAY_FROM_ZERO'",
    "narrow_range: bool = false",
    "axis: int = -1",
    "ensure_minimum_range: float = 0.01",
    "dtype: {bfloat16, float} = DT_FLOAT",
    "classic_asymmetric_algorithm: bool = false"};
const char* const k10_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: Tbias",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k10_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k10_attrs[] = {
    "Tinput: {bfloat16, float} = DT_FLOAT",
    "Tfilter: quantizedtype",
    "Tbias: {float, qint32}",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]",
    "mode: {'MIN_COMBINED', 'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "round_mode: {'HALF_AWAY_FROM_ZERO', 'HALF_TO_EVEN'} = 'HALF_AWAY_FROM_ZERO'",
    "narrow_range: bool = false",
    "axis: int = -1",
    "ensure_minimum_range: float = 0.01"};
const char* const k11_inputs[] = {
    "device_inputs: Tdevice_inputs",
    "host_inputs: Thost_inputs"};
const char* const k11_outputs[] = {
    "device_outputs: Tdevice_outputs",
    "host_outputs: Thost_outputs"};
const char* const k11_attrs[] = {
    "Tdevice_inputs: list(type) >= 0 = []",
    "Thost_inputs: list(type) >= 0 = []",
    "Tdevice_outputs: list(type) >= 0 = []",
    "Thost_outputs: list(type) >= 0 = []",
    "T1: quantizedtype",
    "T2: quantizedtype",
    "U: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "Tout: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "adj_x: bool = false",
    "adj_y: bool = false",
    "fused_ops: list(string) = []",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "output_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'"};
const char* const k12_inputs[] = {
    "x: T1",
    "y: T2",
    "min_x: float",
    "max_x: float",
    "min_y: float",
    "max_y: float"};
const char* const k12_outputs[] = {
    "output: Toutput"};
const char* const k12_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Toutput: {bfloat16, float} = DT_FLOAT",
    "adj_x: bool = false",
    "adj_y: bool = false",
    "is_filter_const: bool = false"};
const char* const k13_inputs[] = {
    "values: N * T",
    "axis: Tidx",
    "input_mins:  N * float",
    "input_maxes: N * float"};
const char* const k13_outputs[] = {
    "output: T",
    "output_min: float",
    "output_max: float"};
const char* const k13_attrs[] = {
    "N: int >= 2",
    "T: numbertype",
    "Tidx: {int32, int64} = DT_INT32"};
const char* const k14_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float"};
const char* const k14_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k14_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k15_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k15_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k15_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k16_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float"};
const char* const k16_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k16_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k17_inputs[] = {
    "device_inputs: Tdevice_inputs",
    "host_inputs: Thost_inputs"};
const char* const k17_outputs[] = {
    "device_outputs: Tdevice_outputs",
    "host_outputs: Thost_outputs"};
const char* const k17_attrs[] = {
    "Tinput: quantizedtype = DT_QUINT8",
    "Tfilter: quantizedtype = DT_QINT8",
    "Tbias: {float, qint32} = DT_QINT32",
    "Tsummand: {float, quint8, qint8, qint32, bfloat16}",
    "out_type: {qint8, quint8, qint32, float, bfloat16}",
    "Tdevice_inputs: list(type) >= 0 = []",
    "Thost_inputs: list(type) >= 0",
    "Tdevice_outputs: list(type) >= 0 = []",
    "Thost_outputs: list(type) >= 0",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "dilations: list(int) = [1, 1, 1, 1]",
    "fused_ops: list(string) = []",
    "alpha: float = 0.0"};
const char* const k18_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: float",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float"};
const char* const k18_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k18_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k19_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: float",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float"};
const char* const k19_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k19_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k20_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: Tbias",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k20_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k20_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "Tbias: {float, qint32}",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k21_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: Tbias",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k21_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k21_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "Tbias: {float, qint32}",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k22_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: Tbias",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float",
    "min_freezed_output: float",
    "max_freezed_output: float",
    "summand: Tsummand",
    "min_summand: float",
    "max_summand: float"};
const char* const k22_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k22_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "Tbias: {float, qint32}",
    "Tsummand: quantizedtype",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k23_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: Tbias",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float",
    "min_freezed_output: float",
    "max_freezed_output: float",
    "summand: Tsummand",
    "min_summand: float",
    "max_summand: float"};
const char* const k23_outputs[] = {
    "output: out_type",
    "min_output: float",
    "max_output: float"};
const char* const k23_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "Tbias: {float, qint32}",
    "Tsummand: quantizedtype",
    "out_type: quantizedtype = DT_QINT32",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k24_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: Tbias",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k24_outputs[] = {
    "output: out_type"};
const char* const k24_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "Tbias: {float, qint32}",
    "out_type: {bfloat16, half} = DT_HALF",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k25_inputs[] = {
    "input: Tinput",
    "filter: Tfilter",
    "bias: Tbias",
    "min_input: float",
    "max_input: float",
    "min_filter: float",
    "max_filter: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k25_outputs[] = {
    "output: out_type"};
const char* const k25_attrs[] = {
    "Tinput: quantizedtype",
    "Tfilter: quantizedtype",
    "Tbias: {float, qint32}",
    "out_type: {bfloat16, half, float} = DT_FLOAT",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "padding_list: list(int) = []",
    "dilations: list(int) = [1, 1, 1, 1]"};
const char* const k26_inputs[] = {
    "x: T1",
    "y: T2",
    "args: num_args * T",
    "min_x: float",
    "max_x: float",
    "min_y: float",
    "max_y: float"};
const char* const k26_outputs[] = {
    "output: Toutput"};
const char* const k26_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "T: {bfloat16, float} = DT_FLOAT",
    "Toutput: {bfloat16, float} = DT_FLOAT",
    "adj_x: bool = false",
    "adj_y: bool = false",
    "num_args: int >= 0",
    "fused_ops: list(string) = []",
    "is_filter_const: bool = false"};
const char* const k27_inputs[] = {
    "a: T1",
    "b: T2",
    "args: num_args * Targs",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float"};
const char* const k27_outputs[] = {
    "product: Toutput",
    "min_product: float",
    "max_product: float"};
const char* const k27_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "num_args: int >= 0",
    "Targs: {bfloat16, half, float, quantizedtype}",
    "Toutput: quantizedtype",
    "T: numbertype",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "fused_ops: list(string) = []",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "epsilon: float = 0.0001",
    "leakyrelu_alpha: float = 0.2",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'"};
const char* const k28_inputs[] = {
    "a: T1",
    "b: T2",
    "args: num_args * Targs",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float"};
const char* const k28_outputs[] = {
    "product: Toutput"};
const char* const k28_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "num_args: int >= 0",
    "Targs: {bfloat16, half, float, quantizedtype}",
    "Toutput: {bfloat16, half, float} = DT_FLOAT",
    "T: numbertype",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "fused_ops: list(string) = []",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "epsilon: float = 0.0001",
    "leakyrelu_alpha: float = 0.2",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'"};
const char* const k29_inputs[] = {
    "a: T1",
    "b: T2",
    "args: num_args * Targs",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k29_outputs[] = {
    "product: Toutput",
    "min_product: float",
    "max_product: float"};
const char* const k29_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "num_args: int >= 0",
    "Targs: {bfloat16, half, float, quantizedtype}",
    "Toutput: quantizedtype",
    "T: numbertype",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "fused_ops: list(string) = []",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "epsilon: float = 0.0001",
    "leakyrelu_alpha: float = 0.2",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'"};
const char* const k30_inputs[] = {
    "device_inputs: Tdevice_inputs",
    "host_inputs: Thost_inputs"};
const char* const k30_outputs[] = {
    "device_outputs: Tdevice_outputs",
    "host_outputs: Thost_outputs"};
const char* const k30_attrs[] = {
    "Tdevice_inputs: list(type) >= 0 = []",
    "Thost_inputs: list(type) >= 0 = []",
    "Tdevice_outputs: list(type) >= 0 = []",
    "Thost_outputs: list(type) >= 0 = []",
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Tbias: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "U: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "Tout: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "is_weight_const: bool = true",
    "is_bias_const: bool = true",
    "fused_ops: list(string) = []",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "output_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "leakyrelu_alpha: float = 0.2"};
const char* const k31_inputs[] = {
    "a: T1",
    "b: T2",
    "bias: Tbias",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float"};
const char* const k31_outputs[] = {
    "out: Toutput",
    "min_out: float",
    "max_out: float"};
const char* const k31_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Tbias: {float, qint32}",
    "Toutput: quantizedtype = DT_QINT32",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'MIN_FIRST'",
    "is_weight_const: bool = true"};
const char* const k32_inputs[] = {
    "a: T1",
    "b: T2",
    "bias: Tbias",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k32_outputs[] = {
    "out: Toutput"};
const char* const k32_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Tbias: {float, bfloat16, qint32}",
    "Toutput: {float, bfloat16}",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'MIN_FIRST'",
    "is_weight_const: bool = true"};
const char* const k33_inputs[] = {
    "a: T1",
    "b: T2",
    "bias: float",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float"};
const char* const k33_outputs[] = {
    "out: Toutput",
    "min_out: float",
    "max_out: float"};
const char* const k33_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Toutput: quantizedtype = DT_QINT32",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'MIN_FIRST'",
    "is_weight_const: bool = true"};
const char* const k34_inputs[] = {
    "a: T1",
    "b: T2",
    "bias: Tbias",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k34_outputs[] = {
    "out: Toutput",
    "min_out: float",
    "max_out: float"};
const char* const k34_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Tbias: {float, qint32}",
    "Toutput: quantizedtype = DT_QUINT8",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'MIN_FIRST'",
    "is_weight_const: bool = true"};
const char* const k35_inputs[] = {
    "a: T1",
    "b: T2",
    "bias: Tbias",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k35_outputs[] = {
    "out: Toutput",
    "min_out: float",
    "max_out: float"};
const char* const k35_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Tbias: {float, qint32}",
    "Toutput: quantizedtype = DT_QUINT8",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'MIN_FIRST'",
    "is_weight_const: bool = true"};
const char* const k36_inputs[] = {
    "input: T",
    "min_input: float",
    "max_input: float"};
const char* const k36_outputs[] = {
    "output: T",
    "min_output: float",
    "max_output: float"};
const char* const k36_attrs[] = {
    "T: quantizedtype",
    "ksize: list(int) >= 4",
    "strides: list(int) >= 4"};
const char* const k37_inputs[] = {
    "tensor: T",
    "shape: Tshape",
    "input_min: float",
    "input_max: float"};
const char* const k37_outputs[] = {
    "output: T",
    "output_min: float",
    "output_max: float"};
const char* const k37_attrs[] = {
    "T: type",
    "Tshape: {int32, int64} = DT_INT32"};
const char* const k38_inputs[] = {
    "x: T",
    "perm: Tperm",
    "min_x: float",
    "max_x: float"};
const char* const k38_outputs[] = {
    "y: T",
    "min_y: float",
    "max_y: float"};
const char* const k38_attrs[] = {
    "T: quantizedtype",
    "Tperm: {int32, int64} = DT_INT32"};
const char* const k39_inputs[] = {
    "device_inputs: Tdevice_inputs",
    "host_inputs: Thost_inputs"};
const char* const k39_outputs[] = {
    "device_outputs: Tdevice_outputs",
    "host_outputs: Thost_outputs"};
const char* const k39_attrs[] = {
    "Tdevice_inputs: list(type) >= 0 = []",
    "Thost_inputs: list(type) >= 0 = []",
    "Tdevice_outputs: list(type) >= 0 = []",
    "Thost_outputs: list(type) >= 0 = []",
    "T1: quantizedtype",
    "T2: quantizedtype",
    "U: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "Tout: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "adj_x: bool = false",
    "adj_y: bool = false",
    "fused_ops: list(string) = []",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "output_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'"};
const char* const k40_inputs[] = {
    "x: T1",
    "y: T2",
    "min_x: float",
    "max_x: float",
    "min_y: float",
    "max_y: float"};
const char* const k40_outputs[] = {
    "output: Toutput"};
const char* const k40_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Toutput: {bfloat16, half, float} = DT_FLOAT",
    "adj_x: bool = false",
    "adj_y: bool = false",
    "is_filter_const: bool = false"};
const char* const k41_inputs[] = {
    "device_inputs: Tdevice_inputs",
    "host_inputs: Thost_inputs"};
const char* const k41_outputs[] = {
    "device_outputs: Tdevice_outputs",
    "host_outputs: Thost_outputs"};
const char* const k41_attrs[] = {
    "Tinput: quantizedtype = DT_QUINT8",
    "Tfilter: quantizedtype = DT_QINT8",
    "Tbias: {float, qint32} = DT_QINT32",
    "Tsummand: {float, quint8, qint8, qint32, bfloat16}",
    "out_type: {qint8, quint8, qint32, float, bfloat16}",
    "Tdevice_inputs: list(type) >= 0 = []",
    "Thost_inputs: list(type) >= 0",
    "Tdevice_outputs: list(type) >= 0 = []",
    "Thost_outputs: list(type) >= 0",
    "data_format: string = 'NHWC'",
    "strides: list(int)",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "dilations: list(int) = [1, 1, 1, 1]",
    "fused_ops: list(string) = []",
    "alpha: float = 0.0"};
const char* const k42_inputs[] = {
    "x: T1",
    "y: T2",
    "args: num_args * T",
    "min_x: float",
    "max_x: float",
    "min_y: float",
    "max_y: float"};
const char* const k42_outputs[] = {
    "output: Toutput"};
const char* const k42_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "T: {bfloat16, half, float} = DT_FLOAT",
    "Toutput: {bfloat16, half, float} = DT_FLOAT",
    "adj_x: bool = false",
    "adj_y: bool = false",
    "num_args: int >= 0",
    "fused_ops: list(string) = []",
    "is_filter_const: bool = false"};
const char* const k43_inputs[] = {
    "a: T1",
    "b: T2",
    "args: num_args * Targs",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float"};
const char* const k43_outputs[] = {
    "product: Toutput",
    "min_product: float",
    "max_product: float"};
const char* const k43_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "num_args: int >= 0",
    "Targs: {float, bfloat16, half, quantizedtype}",
    "Toutput: quantizedtype",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "fused_ops: list(string) = []",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "epsilon: float = 0.0001",
    "leakyrelu_alpha: float = 0.2",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'"};
const char* const k44_inputs[] = {
    "a: T1",
    "b: T2",
    "args: num_args * Targs",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float"};
const char* const k44_outputs[] = {
    "product: Toutput"};
const char* const k44_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "num_args: int >= 0",
    "Targs: {float, bfloat16, half, quantizedtype}",
    "Toutput: {float, bfloat16, half} = DT_FLOAT",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "fused_ops: list(string) = []",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "epsilon: float = 0.0001",
    "leakyrelu_alpha: float = 0.2",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'"};
const char* const k45_inputs[] = {
    "a: T1",
    "b: T2",
    "args: num_args * Targs",
    "min_a: float",
    "max_a: float",
    "min_b: float",
    "max_b: float",
    "min_freezed_output: float",
    "max_freezed_output: float"};
const char* const k45_outputs[] = {
    "product: Toutput",
    "min_product: float",
    "max_product: float"};
const char* const k45_attrs[] = {
    "T1: quantizedtype",
    "T2: quantizedtype",
    "num_args: int >= 0",
    "Targs: {float, bfloat16, half, quantizedtype}",
    "Toutput: quantizedtype",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "fused_ops: list(string) = []",
    "is_filter_const: bool = true",
    "is_bias_const: bool = true",
    "epsilon: float = 0.0001",
    "leakyrelu_alpha: float = 0.2",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'"};
const char* const k46_inputs[] = {
    "device_inputs: Tdevice_inputs",
    "host_inputs: Thost_inputs"};
const char* const k46_outputs[] = {
    "device_outputs: Tdevice_outputs",
    "host_outputs: Thost_outputs"};
const char* const k46_attrs[] = {
    "Tdevice_inputs: list(type) >= 0 = []",
    "Thost_inputs: list(type) >= 0 = []",
    "Tdevice_outputs: list(type) >= 0 = []",
    "Thost_outputs: list(type) >= 0 = []",
    "T1: quantizedtype",
    "T2: quantizedtype",
    "Tbias: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "U: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "Tout: {bfloat16, float, quantizedtype} = DT_FLOAT",
    "transpose_a: bool = false",
    "transpose_b: bool = false",
    "is_weight_const: bool = true",
    "is_bias_const: bool = true",
    "fused_ops: list(string) = []",
    "input_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "output_quant_mode: {'MIN_FIRST', 'SCALED'} = 'SCALED'",
    "leakyrelu_alpha: float = 0.2"};
const char* const k47_inputs[] = {
    "x: T",
    "perm: Tperm",
    "min_x: float",
    "max_x: float"};
const char* const k47_outputs[] = {
    "y: T",
    "min_y: float",
    "max_y: float"};
const char* const k47_attrs[] = {
    "T: quantizedtype",
    "Tperm: {int32, int64} = DT_INT32"};

const OpDefEntry kOpDefs[] = {
    {"Fp8Dequantize", k0_inputs, 2, k0_outputs, 1, k0_attrs, 3},
    {"Fp8Gelu", k1_inputs, 3, k1_outputs, 1, k1_attrs, 3},
    {"Fp8LayerNorm", k2_inputs, 5, k2_outputs, 3, k2_attrs, 6},
    {"Fp8Matmul", k3_inputs, 8, k3_outputs, 1, k3_attrs, 12},
    {"Fp8Quantize", k4_inputs, 3, k4_outputs, 1, k4_attrs, 3},
    {"Fp8QuantizeDbias", k5_inputs, 3, k5_outputs, 2, k5_attrs, 3},
    {"Fp8QuantizeDbiasDgelu", k6_inputs, 4, k6_outputs, 2, k6_attrs, 4},
    {"ITEXQuantizedAvgPool", k7_inputs, 3, k7_outputs, 3, k7_attrs, 3},
    {"_ITEXDequantize", k8_inputs, 3, k8_outputs, 1, k8_attrs, 5},
    {"_ITEXQuantizeV2", k9_inputs, 3, k9_outputs, 3, k9_attrs, 8},
    {"_ITEXQuantizeV2WithQuantizedConv2D", k10_inputs, 9, k10_outputs, 3, k10_attrs, 15},
    {"_ITEXQuantizedBatchMatMul", k11_inputs, 2, k11_outputs, 2, k11_attrs, 13},
    {"_ITEXQuantizedBatchMatMulV2AndDequantize", k12_inputs, 6, k12_outputs, 1, k12_attrs, 6},
    {"_ITEXQuantizedConcatV2", k13_inputs, 4, k13_outputs, 3, k13_attrs, 3},
    {"_ITEXQuantizedConv2D", k14_inputs, 6, k14_outputs, 3, k14_attrs, 8},
    {"_ITEXQuantizedConv2DAndRequantize", k15_inputs, 8, k15_outputs, 3, k15_attrs, 8},
    {"_ITEXQuantizedConv2DPerChannel", k16_inputs, 6, k16_outputs, 3, k16_attrs, 8},
    {"_ITEXQuantizedConv2DV2", k17_inputs, 2, k17_outputs, 2, k17_attrs, 16},
    {"_ITEXQuantizedConv2DWithBias", k18_inputs, 7, k18_outputs, 3, k18_attrs, 9},
    {"_ITEXQuantizedConv2DWithBiasAndRelu", k19_inputs, 7, k19_outputs, 3, k19_attrs, 9},
    {"_ITEXQuantizedConv2DWithBiasAndReluAndRequantize", k20_inputs, 9, k20_outputs, 3, k20_attrs, 10},
    {"_ITEXQuantizedConv2DWithBiasAndRequantize", k21_inputs, 9, k21_outputs, 3, k21_attrs, 10},
    {"_ITEXQuantizedConv2DWithBiasSignedSumAndReluAndRequantize", k22_inputs, 12, k22_outputs, 3, k22_attrs, 11},
    {"_ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize", k23_inputs, 12, k23_outputs, 3, k23_attrs, 11},
    {"_ITEXQuantizedConv2DWithCast", k24_inputs, 9, k24_outputs, 1, k24_attrs, 10},
    {"_ITEXQuantizedConv2DWithDequantize", k25_inputs, 9, k25_outputs, 1, k25_attrs, 10},
    {"_ITEXQuantizedFusedBatchMatMulV2AndDequantize", k26_inputs, 7, k26_outputs, 1, k26_attrs, 9},
    {"_ITEXQuantizedFusedMatMul", k27_inputs, 7, k27_outputs, 3, k27_attrs, 14},
    {"_ITEXQuantizedFusedMatMulAndDequantize", k28_inputs, 7, k28_outputs, 1, k28_attrs, 14},
    {"_ITEXQuantizedFusedMatMulAndRequantize", k29_inputs, 9, k29_outputs, 3, k29_attrs, 14},
    {"_ITEXQuantizedMatMul", k30_inputs, 2, k30_outputs, 2, k30_attrs, 17},
    {"_ITEXQuantizedMatMulWithBias", k31_inputs, 7, k31_outputs, 3, k31_attrs, 8},
    {"_ITEXQuantizedMatMulWithBiasAndDequantize", k32_inputs, 9, k32_outputs, 1, k32_attrs, 8},
    {"_ITEXQuantizedMatMulWithBiasAndRelu", k33_inputs, 7, k33_outputs, 3, k33_attrs, 7},
    {"_ITEXQuantizedMatMulWithBiasAndReluAndRequantize", k34_inputs, 9, k34_outputs, 3, k34_attrs, 8},
    {"_ITEXQuantizedMatMulWithBiasAndRequantize", k35_inputs, 9, k35_outputs, 3, k35_attrs, 8},
    {"_ITEXQuantizedMaxPool", k36_inputs, 3, k36_outputs, 3, k36_attrs, 3},
    {"_ITEXQuantizedReshape", k37_inputs, 4, k37_outputs, 3, k37_attrs, 2},
    {"_ITEXQuantizedTranspose", k38_inputs, 4, k38_outputs, 3, k38_attrs, 2},
    {"_QuantizedBatchMatMul", k39_inputs, 2, k39_outputs, 2, k39_attrs, 13},
    {"_QuantizedBatchMatMulV2AndDequantize", k40_inputs, 6, k40_outputs, 1, k40_attrs, 6},
    {"_QuantizedConv2D", k41_inputs, 2, k41_outputs, 2, k41_attrs, 16},
    {"_QuantizedFusedBatchMatMulV2AndDequantize", k42_inputs, 7, k42_outputs, 1, k42_attrs, 9},
    {"_QuantizedFusedMatMul", k43_inputs, 7, k43_outputs, 3, k43_attrs, 13},
    {"_QuantizedFusedMatMulAndDequantize", k44_inputs, 7, k44_outputs, 1, k44_attrs, 13},
    {"_QuantizedFusedMatMulAndRequantize", k45_inputs, 9, k45_outputs, 3, k45_attrs, 13},
    {"_QuantizedMatMul", k46_inputs, 2, k46_outputs, 2, k46_attrs, 17},
    {"_QuantizedTranspose", k47_inputs, 4, k47_outputs, 3, k47_attrs, 2},
};

}  // namespace
}  // namespace itexb

using namespace itexb;

// Names without a definition of their own: TensorFlow's ops (QuantizeV2, QuantizedConv2DWithBias..., _QuantizedMatMul ...)
// and three names the reference registers kernels for without defining them.  Their argument names - which a plugin
// needs for TF_KernelBuilder_HostMemory - are those of the twin op the reference defines with the same argument list.
static const OpDefEntry* Find(const std::string& name) {
  for (const OpDefEntry& e : kOpDefs)
    if (name == e.name) return &e;
  return nullptr;
}
static const OpDefEntry* FindTwin(const std::string& name) {
  static const char* const kAlias[][2] = {
      {"QuantizedAvgPool", "ITEXQuantizedAvgPool"},
      {"_ITEXQuantizedAvgPool", "ITEXQuantizedAvgPool"},
      {"QuantizedConv2DAndRelu", "_ITEXQuantizedConv2D"},
      {"_ITEXQuantizedConv2DAndRelu", "_ITEXQuantizedConv2D"},
      {"QuantizedConv2DAndReluAndRequantize", "_ITEXQuantizedConv2DAndRequantize"},
      {"_ITEXQuantizedConv2DAndReluAndRequantize", "_ITEXQuantizedConv2DAndRequantize"},
      {"QuantizedConv2DWithBiasSignedSumAndReluAndRequantize", "_ITEXQuantizedConv2DWithBiasSumAndReluAndRequantize"},
  };
  for (const auto& a : kAlias)
    if (name == a[0]) return Find(a[1]);
  if (name.rfind("_Quantized", 0) == 0) return Find("_ITEX" + name.substr(1));  // _QuantizedMatMul -> _ITEXQuantizedMatMul
  return Find("_ITEX" + name);                                                   // QuantizeV2 -> _ITEXQuantizeV2
}

extern "C" int itexb_op_def(const char* op_name, itexb_op_def_t* def) {
  ITEXB_REQUIRE(op_name != nullptr && def != nullptr, ITEXB_INVALID_ARGUMENT, "op_def: NULL argument");
  std::memset(def, 0, sizeof(*def));
  int nin = 0, nout = 0;
  uint32_t hin = 0, hout = 0;
  ITEXB_RETURN_IF_ERROR(itexb_op_signature(op_name, &nin, &nout, &hin, &hout));  // NOT_FOUND for names this library does not implement
  const OpDefEntry* e = Find(op_name);
  def->defined_by_plugin = e != nullptr ? 1 : 0;
  if (e == nullptr) e = FindTwin(op_name);
  def->name = op_name;
  if (e == nullptr) return ITEXB_OK;
  if (def->defined_by_plugin) def->name = e->name;
  def->inputs = e->inputs;
  def->num_inputs = e->num_inputs;
  def->outputs = e->outputs;
  def->num_outputs = e->num_outputs;
  def->attrs = e->attrs;
  def->num_attrs = e->num_attrs;
  return ITEXB_OK;
}
