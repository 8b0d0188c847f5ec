/*
 * OMTensor / OMTensorList as laid out by onnx-mlir's C runtime, implemented
 * independently so that libomcuda can read the wrappers a compiled model
 * passes through krnl.call and so that host programs can link libomcuda
 * alone.  Field order and meaning follow src/Runtime/OMTensor.inc:72-141 and
 * src/Runtime/OMTensorList.inc:35-75 of the onnx-mlir tree; the behaviour of
 * each function follows the lines named in include/omcuda_runtime_abi.h.
 */
#include "omcuda_runtime_abi.h"

#include <stdbool.h>
#include <stdlib.h>
#include <string.h>

struct OMTensor {
  void *allocated;   /* buffer as returned by the allocator */
  void *aligned;     /* first element; what the generated code indexes */
  int64_t offset;    /* always 0 in onnx-mlir */
  int64_t *shape;    /* rank entries */
  int64_t *strides;  /* rank entries, in elements */
  int64_t rank;
  OM_DATA_TYPE dtype;
  int64_t owning;    /* free(allocated) on destroy when non-zero */
};

struct OMTensorList {
  OMTensor **items;
  int64_t size;
  bool shallow; /* only used by the reference's C++ twin; kept for layout */
};

static int64_t dtype_size(OM_DATA_TYPE t) {
  switch (t) {
  case ONNX_TYPE_UINT8:
  case ONNX_TYPE_INT8:
  case ONNX_TYPE_BOOL:
    return 1;
  case ONNX_TYPE_UINT16:
  case ONNX_TYPE_INT16:
  case ONNX_TYPE_FLOAT16:
  case ONNX_TYPE_BFLOAT16:
    return 2;
  case ONNX_TYPE_FLOAT:
  case ONNX_TYPE_INT32:
  case ONNX_TYPE_UINT32:
    return 4;
  case ONNX_TYPE_INT64:
  case ONNX_TYPE_UINT64:
  case ONNX_TYPE_DOUBLE:
  case ONNX_TYPE_COMPLEX64:
  case ONNX_TYPE_STRING:
    return 8;
  case ONNX_TYPE_COMPLEX128:
    return 16;
  default:
    return 0;
  }
}

static OMTensor *alloc_header(int64_t rank) {
  OMTensor *t = (OMTensor *)calloc(1, sizeof(OMTensor));
  if (!t)
    return NULL;
  /* malloc(0) may return NULL; keep one slot so rank-0 tensors stay valid. */
  size_t n = (size_t)(rank > 0 ? rank : 1);
  t->shape = (int64_t *)malloc(n * sizeof(int64_t));
  t->strides = (int64_t *)malloc(n * sizeof(int64_t));
  if (!t->shape || !t->strides) {
    free(t->shape);
    free(t->strides);
    free(t);
    return NULL;
  }
  t->rank = rank;
  t->dtype = ONNX_TYPE_UNDEFINED;
  return t;
}

OMTensor *omTensorCreateUntyped(int64_t rank) { return alloc_header(rank); }

OMTensor *omTensorCreate(
    void *data_ptr, const int64_t *shape, int64_t rank, OM_DATA_TYPE dtype) {
  OMTensor *t = alloc_header(rank);
  if (!t)
    return NULL;
  t->allocated = data_ptr;
  t->aligned = data_ptr;
  t->dtype = dtype;
  int64_t run = 1;
  for (int64_t i = rank - 1; i >= 0; --i) {
    t->shape[i] = shape[i];
    t->strides[i] = run;
    run *= shape[i];
  }
  return t;
}

OMTensor *omTensorCreateWithOwnership(void *data_ptr, const int64_t *shape,
    int64_t rank, OM_DATA_TYPE dtype, int64_t owning) {
  OMTensor *t = omTensorCreate(data_ptr, shape, rank, dtype);
  if (t)
    t->owning = owning;
  return t;
}

OMTensor *omTensorCreateEmpty(
    const int64_t *shape, int64_t rank, OM_DATA_TYPE dtype) {
  int64_t esz = dtype_size(dtype);
  if (esz == 0)
    return NULL;
  int64_t n = 1;
  for (int64_t i = 0; i < rank; ++i)
    n *= shape[i];
  void *buf = malloc((size_t)(n * esz > 0 ? n * esz : 1));
  if (!buf)
    return NULL;
  OMTensor *t = omTensorCreateWithOwnership(buf, shape, rank, dtype, 1);
  if (!t)
    free(buf);
  return t;
}

void omTensorDestroy(OMTensor *t) {
  if (!t)
    return;
  if (t->owning)
    free(t->allocated);
  free(t->shape);
  free(t->strides);
  free(t);
}

void *omTensorGetDataPtr(const OMTensor *t) { return t ? t->aligned : NULL; }

void *omTensorGetAllocatedPtr(const OMTensor *t) {
  return t ? t->allocated : NULL;
}

void omTensorSetDataPtr(
    OMTensor *t, int64_t owning, void *allocatedPtr, void *alignedPtr) {
  if (!t)
    return;
  if (t->owning)
    free(t->allocated);
  t->owning = owning;
  t->allocated = allocatedPtr;
  t->aligned = alignedPtr ? alignedPtr : allocatedPtr;
}

const int64_t *omTensorGetShape(const OMTensor *t) {
  return t ? t->shape : NULL;
}

void omTensorSetShape(OMTensor *t, const int64_t *shape) {
  if (!t || !shape)
    return;
  memcpy(t->shape, shape, (size_t)t->rank * sizeof(int64_t));
}

const int64_t *omTensorGetStrides(const OMTensor *t) {
  return t ? t->strides : NULL;
}

void omTensorSetStrides(OMTensor *t, const int64_t *strides) {
  if (!t || !strides)
    return;
  memcpy(t->strides, strides, (size_t)t->rank * sizeof(int64_t));
}

OM_DATA_TYPE omTensorGetDataType(const OMTensor *t) {
  return t ? t->dtype : ONNX_TYPE_UNDEFINED;
}

void omTensorSetDataType(OMTensor *t, OM_DATA_TYPE dataType) {
  if (t)
    t->dtype = dataType;
}

int64_t omTensorGetNumElems(const OMTensor *t) {
  if (!t)
    return 0;
  int64_t n = 1;
  for (int64_t i = 0; i < t->rank; ++i)
    n *= t->shape[i];
  return n;
}

int64_t omTensorGetBufferSize(const OMTensor *t) {
  return t ? omTensorGetNumElems(t) * dtype_size(t->dtype) : 0;
}

int64_t omTensorGetRank(const OMTensor *t) { return t ? t->rank : 0; }

int64_t omTensorGetOwning(const OMTensor *t) { return t ? t->owning : 0; }

void omTensorSetOwning(OMTensor *t, int64_t owning) {
  if (t)
    t->owning = owning;
}

OMTensorList *omTensorListCreate(OMTensor **tensors, int64_t n) {
  OMTensorList *l = (OMTensorList *)calloc(1, sizeof(OMTensorList));
  if (!l)
    return NULL;
  l->size = n;
  if (n > 0) {
    l->items = (OMTensor **)malloc((size_t)n * sizeof(OMTensor *));
    if (!l->items) {
      free(l);
      return NULL;
    }
    memcpy(l->items, tensors, (size_t)n * sizeof(OMTensor *));
  }
  return l;
}

void omTensorListDestroyShallow(OMTensorList *l) {
  if (!l)
    return;
  free(l->items);
  free(l);
}

void omTensorListDestroy(OMTensorList *l) {
  if (!l)
    return;
  for (int64_t i = 0; i < l->size; ++i)
    omTensorDestroy(l->items[i]);
  omTensorListDestroyShallow(l);
}

OMTensor **omTensorListGetOmtArray(const OMTensorList *l) {
  return l ? l->items : NULL;
}

int64_t omTensorListGetSize(const OMTensorList *l) { return l ? l->size : 0; }

OMTensor *omTensorListGetOmtByIndex(const OMTensorList *l, int64_t index) {
  if (!l || index < 0 || index >= l->size)
    return NULL;
  return l->items[index];
}
