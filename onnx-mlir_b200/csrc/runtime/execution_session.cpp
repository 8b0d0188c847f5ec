// A loader for compiled models: the part of onnx-mlir's ExecutionSession
// (src/Runtime/ExecutionSession.cpp:60-380) that a host program uses to open a
// model .so and call its entry point, as a C API, and aware of device-resident
// tensors: whatever OMTensors the caller passes (host memory, pinned host
// memory, or device memory made with omcudaTensorCreateOnDevice) reach the
// model unchanged, and a model compiled with the CUDA accelerator returns its
// outputs on the side its inputs were on.
//
// Same conventions as the reference: the tag selects the suffixed symbols
// (run_main_graph_<tag>, omQueryEntryPoints_<tag>, ...; "NONE" selects the
// unsuffixed ones; an empty tag means the file name without its extension, in
// lower case), OM_CONSTANT_PATH is set to the model's folder before dlopen
// unless the caller set it (ExecutionSession.cpp:78-92), and a failed run
// returns NULL with errno set (ExecutionSession.cpp:324-362).
//
// Also the external-constants loader a compiled model calls for its
// .constants.bin (src/Runtime/OMExternalConstant.c:57-138): same lookup rule
// (OM_CONSTANT_PATH), mapped read-only.
#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../common.cuh"

using namespace omcuda;

struct omcudaSession {
  void *handle = nullptr;
  std::string path, tag, entry;
  typedef OMTensorList *(*EntryFn)(OMTensorList *);
  typedef const char *const *(*QueryFn)(int64_t *);
  typedef const char *(*SigFn)(const char *);
  EntryFn run = nullptr;
  QueryFn query = nullptr;
  SigFn in_sig = nullptr, out_sig = nullptr;
};

namespace {

std::string lower_stem(const std::string &path) {
  size_t slash = path.find_last_of('/');
  std::string name = slash == std::string::npos ? path : path.substr(slash + 1);
  size_t dot = name.find_last_of('.');
  if (dot != std::string::npos)
    name = name.substr(0, dot);
  std::transform(name.begin(), name.end(), name.begin(),
      [](unsigned char c) { return (char)tolower(c); });
  return name;
}

} // namespace

extern "C" omcudaSession *omcudaSessionCreate(
    const char *shared_lib_path, const char *tag, int default_entry_point) {
  if (!shared_lib_path) {
    fail(OMCUDA_EINVAL, "SessionCreate: null path");
    return nullptr;
  }
  std::string path = shared_lib_path;
  // The model's constructor looks its constants file up in OM_CONSTANT_PATH
  // while dlopen runs: point it at the model's folder for that long, unless
  // the caller chose a folder.
  bool set_constant_path = false;
  if (!getenv("OM_CONSTANT_PATH")) {
    size_t slash = path.find_last_of('/');
    setenv("OM_CONSTANT_PATH", slash == std::string::npos ? "." : path.substr(0, slash).c_str(),
        /*overwrite=*/0);
    set_constant_path = true;
  }
  std::string t = (tag && *tag) ? tag : lower_stem(path);
  std::string suffix = strcasecmp(t.c_str(), "NONE") == 0 ? "" : "_" + t;
  void *h = dlopen(path.c_str(), RTLD_LAZY | RTLD_GLOBAL);
  if (set_constant_path)
    unsetenv("OM_CONSTANT_PATH");
  if (!h) {
    fail(OMCUDA_EINVAL, "SessionCreate: cannot open library '%s': %s", path.c_str(), dlerror());
    return nullptr;
  }
  omcudaSession *s = new omcudaSession();
  s->handle = h;
  s->path = path;
  s->tag = t;
  auto sym = [&](const char *base) { return dlsym(h, (std::string(base) + suffix).c_str()); };
  s->query = (omcudaSession::QueryFn)sym("omQueryEntryPoints");
  s->in_sig = (omcudaSession::SigFn)sym("omInputSignature");
  s->out_sig = (omcudaSession::SigFn)sym("omOutputSignature");
  if (!s->query || !s->in_sig || !s->out_sig) {
    fail(OMCUDA_EINVAL, "SessionCreate: cannot load symbol 'omQueryEntryPoints%s' (or the "
                        "signature functions) from '%s'", suffix.c_str(), path.c_str());
    dlclose(h);
    delete s;
    return nullptr;
  }
  if (default_entry_point) {
    s->entry = "run_main_graph" + suffix;
    s->run = (omcudaSession::EntryFn)dlsym(h, s->entry.c_str());
    if (!s->run) {
      fail(OMCUDA_EINVAL, "SessionCreate: cannot load symbol '%s'", s->entry.c_str());
      dlclose(h);
      delete s;
      return nullptr;
    }
  }
  return s;
}

extern "C" const char *const *omcudaSessionQueryEntryPoints(
    omcudaSession *s, int64_t *num_entry_points) {
  if (!s)
    return nullptr;
  return s->query(num_entry_points);
}

extern "C" int omcudaSessionSetEntryPoint(omcudaSession *s, const char *name) {
  if (!s || !name)
    return fail(OMCUDA_EINVAL, "SessionSetEntryPoint: null argument");
  void *f = dlsym(s->handle, name);
  if (!f)
    return fail(OMCUDA_EINVAL, "SessionSetEntryPoint: cannot load symbol '%s'", name);
  s->run = (omcudaSession::EntryFn)f;
  s->entry = name;
  return OMCUDA_OK;
}

extern "C" const char *omcudaSessionInputSignature(omcudaSession *s) {
  if (!s || !s->run) {
    fail(OMCUDA_EINVAL, "SessionInputSignature: no entry point set");
    return nullptr;
  }
  return s->in_sig(s->entry.c_str());
}

extern "C" const char *omcudaSessionOutputSignature(omcudaSession *s) {
  if (!s || !s->run) {
    fail(OMCUDA_EINVAL, "SessionOutputSignature: no entry point set");
    return nullptr;
  }
  return s->out_sig(s->entry.c_str());
}

extern "C" OMTensorList *omcudaSessionRun(omcudaSession *s, OMTensorList *inputs) {
  if (!s || !s->run) {
    fail(OMCUDA_EINVAL, "SessionRun: no entry point set");
    return nullptr;
  }
  if (!inputs) {
    fail(OMCUDA_EINVAL, "SessionRun: null input list");
    return nullptr;
  }
  errno = 0;
  OMTensorList *out = s->run(inputs);
  if (!out && errno == 0)
    errno = EIO; // the model reported failure without a reason
  return out;
}

extern "C" void omcudaSessionDestroy(omcudaSession *s) {
  if (!s)
    return;
  if (s->handle)
    dlclose(s->handle);
  delete s;
}

// ---- external constants ------------------------------------------------------

extern "C" int omcudaLoadConstantData(
    void **const_addr, const char *fname, int64_t size, int64_t is_le) {
  if (!const_addr || !fname)
    return fail(OMCUDA_EINVAL, "LoadConstantData: null pointer");
  if (size <= 0)
    return fail(OMCUDA_EINVAL, "LoadConstantData: file size is zero");
  if (*const_addr)
    return OMCUDA_OK; // already loaded
  const uint16_t probe = 1;
  const bool host_le = *(const uint8_t *)&probe == 1;
  if ((is_le != 0) != host_le)
    return fail(OMCUDA_EINVAL, "LoadConstantData: the constant pack is stored in a byte "
                               "order that is not native to this system");
  std::string path = fname;
  if (const char *base = getenv("OM_CONSTANT_PATH"))
    path = std::string(base) + "/" + fname;
  int fd = open(path.c_str(), O_RDONLY);
  if (fd < 0)
    return fail(OMCUDA_EINVAL, "LoadConstantData: cannot open %s: %s; set OM_CONSTANT_PATH to "
                               "the folder that contains %s", path.c_str(), strerror(errno), fname);
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < size) {
    close(fd);
    return fail(OMCUDA_EINVAL, "LoadConstantData: %s is shorter than the %lld bytes the model "
                               "expects", path.c_str(), (long long)size);
  }
  void *p = mmap(nullptr, (size_t)size, PROT_READ, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED)
    return fail(OMCUDA_ENOMEM, "LoadConstantData: mmap of %s failed: %s", path.c_str(),
        strerror(errno));
  *const_addr = p;
  return OMCUDA_OK;
}

extern "C" int omcudaUnloadConstantData(void **const_addr, int64_t size) {
  if (!const_addr || !*const_addr)
    return OMCUDA_EINVAL;
  munmap(*const_addr, (size_t)size);
  *const_addr = nullptr;
  return OMCUDA_OK;
}
