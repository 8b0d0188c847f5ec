// RUN: onnx-mlir-opt --maccel=CUDA --shape-inference --convert-onnx-to-krnl --canonicalize %s -split-input-file | FileCheck %s

// The fp32 ops a quantized encoder holds between its linears.  Integer
// attributes reach the library as int64_t, float attributes as double, after
// the tensors and in attribute-name order.

func.func @test_softmax_last_axis(%arg0: tensor<32x12x128x128xf32>) -> tensor<32x12x128x128xf32> {
  %0 = "onnx.Softmax"(%arg0) {axis = -1 : si64} : (tensor<32x12x128x128xf32>) -> tensor<32x12x128x128xf32>
  return %0 : tensor<32x12x128x128xf32>

// CHECK-LABEL:  func.func @test_softmax_last_axis
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<32x12x128x128xf32>) -> memref<32x12x128x128xf32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<32x12x128x128xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]]) <{funcName = "omcudaSoftmax", numOfOutput = 1 : si64}> {axis = -1 : si64} : (memref<32x12x128x128xf32>, memref<32x12x128x128xf32>) -> ()
// CHECK:           return [[RES_]] : memref<32x12x128x128xf32>
}

// -----

func.func @test_softmax_other_axis_stays_on_cpu(%arg0: tensor<10x20x30xf32>) -> tensor<10x20x30xf32> {
  %0 = "onnx.Softmax"(%arg0) {axis = 1 : si64} : (tensor<10x20x30xf32>) -> tensor<10x20x30xf32>
  return %0 : tensor<10x20x30xf32>

// CHECK-LABEL:  func.func @test_softmax_other_axis_stays_on_cpu
// CHECK-NOT:       omcudaSoftmax
// CHECK:           krnl.iterate
}

// -----

func.func @test_layernorm(%arg0: tensor<32x128x768xf32>, %arg1: tensor<768xf32>, %arg2: tensor<768xf32>) -> tensor<32x128x768xf32> {
  %y, %mean, %inv = "onnx.LayerNormalization"(%arg0, %arg1, %arg2) {axis = -1 : si64, epsilon = 9.99999974E-6 : f32, stash_type = 1 : si64} : (tensor<32x128x768xf32>, tensor<768xf32>, tensor<768xf32>) -> (tensor<32x128x768xf32>, none, none)
  return %y : tensor<32x128x768xf32>

// CHECK-LABEL:  func.func @test_layernorm
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<32x128x768xf32>, [[PARAM_1_:%.+]]: memref<768xf32>, [[PARAM_2_:%.+]]: memref<768xf32>) -> memref<32x128x768xf32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<32x128x768xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]], [[PARAM_2_]]) <{funcName = "omcudaLayerNormalization", numOfOutput = 1 : si64}> {axis = -1 : si64, epsilon = 9.99999974E-6 : f32} : (memref<32x128x768xf32>, memref<32x128x768xf32>, memref<768xf32>, memref<768xf32>) -> ()
// CHECK:           return [[RES_]] : memref<32x128x768xf32>
}

// -----

func.func @test_gelu_none(%arg0: tensor<4096x3072xf32>) -> tensor<4096x3072xf32> {
  %0 = "onnx.Gelu"(%arg0) {approximate = "none"} : (tensor<4096x3072xf32>) -> tensor<4096x3072xf32>
  return %0 : tensor<4096x3072xf32>

// CHECK-LABEL:  func.func @test_gelu_none
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<4096x3072xf32>) -> memref<4096x3072xf32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<4096x3072xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]]) <{funcName = "omcudaGelu", numOfOutput = 1 : si64}> : (memref<4096x3072xf32>, memref<4096x3072xf32>) -> ()
// CHECK:           return [[RES_]] : memref<4096x3072xf32>
}

// -----

func.func @test_residual_add(%arg0: tensor<32x128x768xf32>, %arg1: tensor<32x128x768xf32>) -> tensor<32x128x768xf32> {
  %0 = "onnx.Add"(%arg0, %arg1) : (tensor<32x128x768xf32>, tensor<32x128x768xf32>) -> tensor<32x128x768xf32>
  return %0 : tensor<32x128x768xf32>

// CHECK-LABEL:  func.func @test_residual_add
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<32x128x768xf32>, [[PARAM_1_:%.+]]: memref<32x128x768xf32>) -> memref<32x128x768xf32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<32x128x768xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]]) <{funcName = "omcudaAdd", numOfOutput = 1 : si64}> : (memref<32x128x768xf32>, memref<32x128x768xf32>, memref<32x128x768xf32>) -> ()
// CHECK:           return [[RES_]] : memref<32x128x768xf32>
}

// -----

func.func @test_transpose_heads(%arg0: tensor<32x128x12x64xf32>) -> tensor<32x12x128x64xf32> {
  %0 = "onnx.Transpose"(%arg0) {perm = [0, 2, 1, 3]} : (tensor<32x128x12x64xf32>) -> tensor<32x12x128x64xf32>
  return %0 : tensor<32x12x128x64xf32>

// CHECK-LABEL:  func.func @test_transpose_heads
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<32x128x12x64xf32>) -> memref<32x12x128x64xf32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<32x12x128x64xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]]) <{funcName = "omcudaTranspose0213", numOfOutput = 1 : si64}> : (memref<32x12x128x64xf32>, memref<32x128x12x64xf32>) -> ()
// CHECK:           return [[RES_]] : memref<32x12x128x64xf32>
}

// -----

func.func @test_matmul_f32_batched(%arg0: tensor<32x12x128x64xf32>, %arg1: tensor<32x12x64x128xf32>) -> tensor<32x12x128x128xf32> {
  %0 = "onnx.MatMul"(%arg0, %arg1) : (tensor<32x12x128x64xf32>, tensor<32x12x64x128xf32>) -> tensor<32x12x128x128xf32>
  return %0 : tensor<32x12x128x128xf32>

// CHECK-LABEL:  func.func @test_matmul_f32_batched
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<32x12x128x64xf32>, [[PARAM_1_:%.+]]: memref<32x12x64x128xf32>) -> memref<32x12x128x128xf32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<32x12x128x128xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]]) <{funcName = "omcudaMatMulF32", numOfOutput = 1 : si64}> : (memref<32x12x128x128xf32>, memref<32x12x128x64xf32>, memref<32x12x64x128xf32>) -> ()
// CHECK:           return [[RES_]] : memref<32x12x128x128xf32>
}

// -----

// onnx.Custom ops made by the accelerator's rewrites go through the stock
// ONNXCustomOpLowering.

func.func @test_custom_dyn_quant_linear(%arg0: tensor<128x768xf32>, %arg1: tensor<768x768xi8>, %arg2: tensor<f32>, %arg3: tensor<768xf32>) -> tensor<128x768xf32> {
  %none = "onnx.NoValue"() {value} : () -> none
  %0 = "onnx.Custom"(%arg0, %arg1, %arg2, %none, %arg3) {function_name = "omcudaDynQuantLinear", scaleForm = 0 : si64, shape_infer_pattern = "MDBroadcast", output_element_type = f32} : (tensor<128x768xf32>, tensor<768x768xi8>, tensor<f32>, none, tensor<768xf32>) -> tensor<128x768xf32>
  return %0 : tensor<128x768xf32>

// CHECK-LABEL:  func.func @test_custom_dyn_quant_linear
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<128x768xf32>, [[PARAM_1_:%.+]]: memref<768x768xi8>, [[PARAM_2_:%.+]]: memref<f32>, [[PARAM_3_:%.+]]: memref<768xf32>) -> memref<128x768xf32> {
// CHECK:           [[VAR_0_:%.+]] = "onnx.NoValue"() {value} : () -> none
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<128x768xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]], [[PARAM_2_]], [[VAR_0_]], [[PARAM_3_]]) <{funcName = "omcudaDynQuantLinear", numOfOutput = 1 : si64}> {scaleForm = 0 : si64} : (memref<128x768xf32>, memref<128x768xf32>, memref<768x768xi8>, memref<f32>, none, memref<768xf32>) -> ()
// CHECK:           return [[RES_]] : memref<128x768xf32>
}

// -----

func.func @test_custom_attention(%arg0: tensor<32x128x768xf32>, %arg1: tensor<32x128x768xf32>, %arg2: tensor<32x128x768xf32>) -> tensor<32x128x768xf32> {
  %0 = "onnx.Custom"(%arg0, %arg1, %arg2) {function_name = "omcudaAttention", heads = 12 : si64, scale = 1.250000e-01 : f32, shape_infer_pattern = "SameAs"} : (tensor<32x128x768xf32>, tensor<32x128x768xf32>, tensor<32x128x768xf32>) -> tensor<32x128x768xf32>
  return %0 : tensor<32x128x768xf32>

// CHECK-LABEL:  func.func @test_custom_attention
// CHECK-SAME:   ([[PARAM_0_:%.+]]: memref<32x128x768xf32>, [[PARAM_1_:%.+]]: memref<32x128x768xf32>, [[PARAM_2_:%.+]]: memref<32x128x768xf32>) -> memref<32x128x768xf32> {
// CHECK:           [[RES_:%.+]] = memref.alloc() {{.*}}: memref<32x128x768xf32>
// CHECK:           "krnl.call"([[RES_]], [[PARAM_0_]], [[PARAM_1_]], [[PARAM_2_]]) <{funcName = "omcudaAttention", numOfOutput = 1 : si64}> {heads = 12 : si64, scale = 1.250000e-01 : f32} : (memref<32x128x768xf32>, memref<32x128x768xf32>, memref<32x128x768xf32>, memref<32x128x768xf32>) -> ()
// CHECK:           return [[RES_]] : memref<32x128x768xf32>
}
