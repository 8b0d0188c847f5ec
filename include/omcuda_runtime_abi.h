/*
 * The slice of onnx-mlir's C runtime ABI that libomcuda implements itself.
 *
 * A model compiled by onnx-mlir links the reference's libcruntime.a and hands
 * `OMTensor *` wrappers to external functions (krnl.call).  libomcuda reads
 * those wrappers, so it carries its own implementation of the struct layout
 * and of the accessor functions, with the same symbol names and signatures as
 * the reference, so that a host program (a loader, a test, the config
 * harnesses) can link libomcuda alone.
 *
 * Layout and semantics follow, in the onnx-mlir tree:
 *   struct OMTensor          src/Runtime/OMTensor.inc:72-141
 *   create / destroy         src/Runtime/OMTensor.inc:166-272
 *   accessors                src/Runtime/OMTensor.inc:274-420
 *   OMTensorList             src/Runtime/OMTensorList.inc:33-140
 *   OM_DATA_TYPE values      include/onnx-mlir/Runtime/OnnxDataTypeMetaData.inc:24-45
 *   public declarations      include/onnx-mlir/Runtime/OMTensor.h:92-358,
 *                            include/onnx-mlir/Runtime/OMTensorList.h:44-99
 *
 * Nothing is appended to the struct: whether a tensor's buffer lives in host
 * or device memory is a property of the pointer (asked of the CUDA driver),
 * not of the wrapper, so wrappers made by an unmodified libcruntime work.
 */
#ifndef OMCUDA_RUNTIME_ABI_H
#define OMCUDA_RUNTIME_ABI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ONNX element types; numeric values are ONNX's TensorProto.DataType. */
typedef enum {
  ONNX_TYPE_UNDEFINED = 0,
  ONNX_TYPE_FLOAT = 1,
  ONNX_TYPE_UINT8 = 2,
  ONNX_TYPE_INT8 = 3,
  ONNX_TYPE_UINT16 = 4,
  ONNX_TYPE_INT16 = 5,
  ONNX_TYPE_INT32 = 6,
  ONNX_TYPE_INT64 = 7,
  ONNX_TYPE_STRING = 8,
  ONNX_TYPE_BOOL = 9,
  ONNX_TYPE_FLOAT16 = 10,
  ONNX_TYPE_DOUBLE = 11,
  ONNX_TYPE_UINT32 = 12,
  ONNX_TYPE_UINT64 = 13,
  ONNX_TYPE_COMPLEX64 = 14,
  ONNX_TYPE_COMPLEX128 = 15,
  ONNX_TYPE_BFLOAT16 = 16
} OM_DATA_TYPE;

typedef struct OMTensor OMTensor;
typedef struct OMTensorList OMTensorList;

/* OMTensor.h:92 — non-owning wrapper over caller memory, dense row-major
 * strides computed from the shape. */
OMTensor *omTensorCreate(
    void *data_ptr, const int64_t *shape, int64_t rank, OM_DATA_TYPE dtype);
/* OMTensor.h:123 */
OMTensor *omTensorCreateWithOwnership(void *data_ptr, const int64_t *shape,
    int64_t rank, OM_DATA_TYPE dtype, int64_t owning);
/* OMTensor.h:143 — malloc'ed, owning host buffer. */
OMTensor *omTensorCreateEmpty(
    const int64_t *shape, int64_t rank, OM_DATA_TYPE dtype);
/* OMTensor.inc:220-240 — used by the generated entry point and by krnl.call. */
OMTensor *omTensorCreateUntyped(int64_t rank);
/* OMTensor.h:159 — frees the buffer with free() only when owning. */
void omTensorDestroy(OMTensor *tensor);
/* OMTensor.h:168,183 */
void *omTensorGetDataPtr(const OMTensor *tensor);
void *omTensorGetAllocatedPtr(const OMTensor *tensor);
/* OMTensor.inc:294-308 */
void omTensorSetDataPtr(
    OMTensor *tensor, int64_t owning, void *allocatedPtr, void *alignedPtr);
/* OMTensor.h:197-245 */
const int64_t *omTensorGetShape(const OMTensor *tensor);
void omTensorSetShape(OMTensor *tensor, const int64_t *shape);
const int64_t *omTensorGetStrides(const OMTensor *tensor);
void omTensorSetStrides(OMTensor *tensor, const int64_t *strides);
/* OMTensor.h:279-347 */
OM_DATA_TYPE omTensorGetDataType(const OMTensor *tensor);
void omTensorSetDataType(OMTensor *tensor, OM_DATA_TYPE dataType);
int64_t omTensorGetBufferSize(const OMTensor *tensor);
int64_t omTensorGetRank(const OMTensor *tensor);
int64_t omTensorGetNumElems(const OMTensor *tensor);
int64_t omTensorGetOwning(const OMTensor *tensor);
void omTensorSetOwning(OMTensor *tensor, int64_t owning);

/* OMTensorList.h:44-99 */
OMTensorList *omTensorListCreate(OMTensor **tensors, int64_t n);
void omTensorListDestroy(OMTensorList *list);
void omTensorListDestroyShallow(OMTensorList *list);
OMTensor **omTensorListGetOmtArray(const OMTensorList *list);
int64_t omTensorListGetSize(const OMTensorList *list);
OMTensor *omTensorListGetOmtByIndex(const OMTensorList *list, int64_t index);

#ifdef __cplusplus
}
#endif
#endif
