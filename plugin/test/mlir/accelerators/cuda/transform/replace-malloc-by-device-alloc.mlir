// RUN: onnx-mlir-opt --maccel=CUDA --replace-malloc-by-omcuda-device-alloc %s | FileCheck %s

// Intermediates of a fully offloaded model move to device memory; a buffer
// that is handed back to the caller as an output OMTensor keeps malloc.

module {
  llvm.func @malloc(i64) -> !llvm.ptr
  llvm.func @free(!llvm.ptr)
  llvm.func @omTensorSetDataPtr(!llvm.ptr, i64, !llvm.ptr, !llvm.ptr)
  llvm.func @omcudaGelu(!llvm.ptr, !llvm.ptr)

  llvm.func @graph(%x: !llvm.ptr, %omt: !llvm.ptr) {
    %size = llvm.mlir.constant(4096 : i64) : i64
    %own = llvm.mlir.constant(1 : i64) : i64
    %tmp = llvm.call @malloc(%size) : (i64) -> !llvm.ptr
    %out = llvm.call @malloc(%size) : (i64) -> !llvm.ptr
    llvm.call @omcudaGelu(%tmp, %x) : (!llvm.ptr, !llvm.ptr) -> ()
    llvm.call @omcudaGelu(%out, %tmp) : (!llvm.ptr, !llvm.ptr) -> ()
    llvm.call @free(%tmp) : (!llvm.ptr) -> ()
    llvm.call @omTensorSetDataPtr(%omt, %own, %out, %out) : (!llvm.ptr, i64, !llvm.ptr, !llvm.ptr) -> ()
    llvm.return
  }

// CHECK-LABEL:  llvm.func @graph
// CHECK:           [[TMP_:%.+]] = llvm.call @omcudaDeviceAlloc({{.*}}) : (i64) -> !llvm.ptr
// CHECK:           [[OUT_:%.+]] = llvm.call @malloc({{.*}}) : (i64) -> !llvm.ptr
// CHECK:           llvm.call @omcudaGelu([[TMP_]], {{.*}}) : (!llvm.ptr, !llvm.ptr) -> ()
// CHECK:           llvm.call @omcudaGelu([[OUT_]], [[TMP_]]) : (!llvm.ptr, !llvm.ptr) -> ()
// CHECK:           llvm.call @omcudaDeviceFree([[TMP_]]) : (!llvm.ptr) -> ()
// CHECK-NOT:       llvm.call @free
// CHECK:           llvm.call @omTensorSetDataPtr({{.*}}, {{.*}}, [[OUT_]], [[OUT_]])
}
