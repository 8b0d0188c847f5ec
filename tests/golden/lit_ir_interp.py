"""A small interpreter for the Krnl-level IR that onnx-mlir's lowering tests
expect (the `// CHECK` lines of test/mlir/conversion/onnx_to_krnl/**).

Those FileCheck expectations are the reference's own statement of what
`convert-onnx-to-krnl` emits for DynamicQuantizeLinear, QuantizeLinear,
DequantizeLinear, MatMulInteger and QLinearMatMul.  Executing them on seeded
inputs gives value-level golden vectors that come from the reference's emitted
op sequence rather than from this repository's reading of it.  Used only by
make_lit_ir_golden.py to (re)generate fixtures; the test-suite reads the
fixtures, not the reference tree.

The fp32 ops of the encoder graphs (Softmax, MatMul, Gelu, LayerNormalization)
are covered the same way; their IR adds math.{exp,erf,sqrt} (evaluated with
the host libm's expf / erff, which is what a compiled model calls,
src/Conversion/KrnlToLLVM/KrnlUnaryMath.cpp:39-45), the vector dialect ops the
SIMD lowering of LayerNormalization uses (vector.{load,store,shuffle,
broadcast}, dense vector constants), scf.for, memref.{load,store} and
krnl.block (loop tiling).

Supported: krnl.global (dense constants), arith.{constant,addf,subf,mulf,divf,minnumf,maxnumf,cmpf,select,
addi,subi,muli,extsi,extui,trunci,sitofp,uitofp,fptosi,fptoui}, math.floor,
builtin.unrealized_conversion_cast, memref.{alloc,dim,reshape,reinterpret_cast}, affine.apply
of the single-result maps these tests use, krnl.{define_loops,iterate (with
and without iter_args),get_induction_var_value,load,store,memset,yield}.
fp32 arithmetic is done with numpy float32 scalars (one rounding per op);
integers wrap to their bit width.
"""
import ctypes
import ctypes.util
import re

import numpy as np

_libm = ctypes.CDLL(ctypes.util.find_library("m"))
for _f in ("expf", "erff"):
    getattr(_libm, _f).restype = ctypes.c_float
    getattr(_libm, _f).argtypes = [ctypes.c_float]


def _libm_map(fn, x):
    """Applies a libm float function to a float32 scalar or vector."""
    if np.ndim(x) == 0:
        return np.float32(fn(float(x)))
    return np.array([fn(float(v)) for v in x], np.float32)

_NP = {"f32": np.float32, "i8": np.int8, "ui8": np.uint8, "i16": np.int16,
       "i32": np.int32, "ui32": np.uint32, "i64": np.int64, "index": np.int64}


def extract_functions(text):
    """Splits a lit file into {func_name: dict(stmts, maps, params, results)}.
    stmts are the normalised CHECK lines of the body; maps the affine maps the
    test names before the function; params / results the memref types of the
    signature, e.g. [("16x32", "i8"), ...]."""
    funcs = {}
    cur = None
    maps = {}
    for raw in text.splitlines():
        m = re.match(r"\s*//\s*CHECK(?:-[A-Z]+)?:\s?(.*)$", raw)
        if not m:
            if re.match(r"\s*//\s*-----", raw):
                cur = None
                maps = {}
            continue
        line = m.group(1).rstrip()
        if "separator of consecutive DAGs" in line:
            continue
        norm = _normalise(line)
        mm = re.match(r"(%\w+)\s*=\s*affine_map<(.*)>$", norm)
        if mm:
            maps[mm.group(1)] = mm.group(2)
            continue
        lab = re.match(r"\s*func\.func (?:private )?@(\w+)", line)
        if lab:
            cur = lab.group(1)
            funcs[cur] = {"stmts": [], "maps": dict(maps), "params": [], "results": [],
                          "param_names": []}
            continue
        if cur is None:
            continue
        if norm.startswith("(") and "->" in norm and not funcs[cur]["params"]:
            sig, res = norm.rsplit("->", 1)
            mt = r"memref<((?:[\d?]+x)*)(\w+)>"
            funcs[cur]["params"] = [(a.rstrip("x"), b) for a, b in re.findall(mt, sig)]
            funcs[cur]["param_names"] = re.findall(r"(%\w+)\s*:\s*memref<", sig)
            funcs[cur]["results"] = [(a.rstrip("x"), b) for a, b in re.findall(mt, res)]
            continue
        funcs[cur]["stmts"].append(norm)
    return funcs


def _normalise(line):
    # [[NAME_:%.+]] and [[NAME_]] -> %NAME_ ; {{.}} -> bracket marker ; drop {{.*}}
    line = re.sub(r"\[\[([A-Za-z0-9_]+):[^\]]*\]\]", r"%\1", line)
    line = re.sub(r"\[\[([A-Za-z0-9_]+)\]\]", r"%\1", line)
    line = line.replace("{{.*}}", " ")
    line = line.replace("{{.}}", "|")
    return line.strip()


class Interp:
    def __init__(self, stmts, maps=None):
        self.stmts = stmts
        self.maps = maps or {}
        self.env = {}
        self.loop_bounds = {}
        self.loop_iv = {}
        self.blocks = {}   # tile loop -> (parent loop, tile size)

    # ---- values ---------------------------------------------------------
    def val(self, tok):
        tok = tok.strip()
        if tok in self.env:
            return self.env[tok]
        if re.fullmatch(r"-?\d+", tok):
            return int(tok)
        raise KeyError("unknown value %r" % tok)

    @staticmethod
    def wrap(v, ty):
        bits = {"i1": 1, "i8": 8, "ui8": 8, "i16": 16, "i32": 32, "i64": 64,
                "index": 64}[ty]
        v = int(v) & ((1 << bits) - 1)
        if not ty.startswith("u") and ty != "i1" and v >= 1 << (bits - 1):
            v -= 1 << bits
        return v

    # ---- execution --------------------------------------------------------
    def run(self, params, names=None):
        """params: list of numpy arrays bound to the signature's names (or to
        %PARAM_0_, %PARAM_1_, ... when no names are given)."""
        for i, a in enumerate(params):
            self.env[names[i] if names else "%%PARAM_%d_" % i] = a
        self.result = None
        self.block(0, len(self.stmts))
        return self.result

    def find_end(self, start):
        depth = 0
        for i in range(start, len(self.stmts)):
            s = self.stmts[i]
            if s.endswith("{"):
                depth += 1
            if s == "}":
                depth -= 1
                if depth == 0:
                    return i
        raise ValueError("unbalanced block at %d" % start)

    def block(self, lo, hi):
        i = lo
        yielded = None
        while i < hi:
            s = self.stmts[i]
            if "krnl.iterate() with ()" in s and s.endswith("{"):
                end = self.find_end(i)      # a loop nest of depth 0: run the body once
                self.block(i + 1, end)
                i = end + 1
                continue
            if "krnl.iterate(" in s and s.endswith("{"):
                end = self.find_end(i)
                self.iterate(s, i + 1, end)
                i = end + 1
                continue
            if s.startswith("scf.for") and s.endswith("{"):
                end = self.find_end(i)
                m = re.match(r"scf\.for (%\w+) = (%?\w+) to (%?\w+) step (%?\w+)", s)
                for v in range(int(self.val(m.group(2))), int(self.val(m.group(3))),
                               int(self.val(m.group(4)))):
                    self.env[m.group(1)] = v
                    self.block(i + 1, end)
                i = end + 1
                continue
            if s.startswith("krnl.yield"):
                yielded = self.val(s.split()[1])
            elif s.startswith("return") or s.startswith("onnx.Return"):
                names = [t.strip() for t in s.split(None, 1)[1].split(":")[0].split(",")]
                self.result = names
            elif s not in ("}", ""):
                self.stmt(s)
            i += 1
        return yielded

    def bound(self, tok):
        tok = tok.strip()
        m = re.match(r"(%\w+)\((.*)\)$", tok)          # MAP(args)
        if m:
            return self.apply_map(m.group(1), [self.val(a) for a in m.group(2).split(",")], [])
        return self.val(tok)

    def iterate(self, header, lo, hi):
        # [%X = ] krnl.iterate(L#0, L#1) with (L#0 -> %I = a to b, ...)
        #         [iter_args(%A = %INIT) -> (ty)] {
        res = None
        m = re.match(r"(%\w+)\s*=\s*krnl\.iterate", header)
        if m:
            res = m.group(1)
        loops = [t.strip() for t in
                 re.search(r"krnl\.iterate\(([^)]*)\)", header).group(1).split(",")]
        with_part = re.search(r"with \((.*?)\)\s*(iter_args|\{)", header).group(1)
        for d in re.finditer(r"(%\w+(?:#\d+)?)\s*->\s*%\w+\s*=\s*(.+?)\s+to\s+"
                             r"((?:%\w+\([^)]*\))|[^,]+)", with_part):
            self.loop_bounds[d.group(1)] = (d.group(2), d.group(3))
        ia = re.search(r"iter_args\((%\w+)\s*=\s*(%?\w+)\)", header)
        acc_name, acc = (ia.group(1), self.val(ia.group(2))) if ia else (None, None)
        ranges = []
        for L in loops:
            # a tile loop made by krnl.block walks its parent's range in steps
            parent, step = self.blocks.get(L, (L, 1))
            a, b = self.loop_bounds[parent]
            ranges.append((L, int(self.bound(a)), int(self.bound(b)), step))

        def rec(k):
            nonlocal acc
            if k == len(ranges):
                if acc_name:
                    self.env[acc_name] = acc
                y = self.block(lo, hi)
                if acc_name:
                    acc = y
                return
            L, a, b, step = ranges[k]
            for v in range(a, b, step):
                self.loop_iv[L] = v
                rec(k + 1)
        rec(0)
        if res:
            self.env[res] = acc

    def apply_map(self, name, dims, syms):
        expr = self.maps[name]
        m = re.match(r"\((.*?)\)(?:\[(.*?)\])?\s*->\s*\((.*)\)", expr)
        dn = [t.strip() for t in m.group(1).split(",") if t.strip()]
        sn = [t.strip() for t in (m.group(2) or "").split(",") if t.strip()]
        scope = dict(zip(dn, dims))
        scope.update(zip(sn, syms))
        body = m.group(3).replace(" floordiv ", " // ").replace(" mod ", " % ")
        return int(eval(body, {"__builtins__": {}}, scope))

    def memref_index(self, s):
        # "%M|%a, %b]" or "%M|%a|" or "%M[]" or "%M[0]" -> (name, idx tuple)
        m = re.match(r"(%\w+)\s*(?:\[|\|)(.*?)(?:\]|\|)?$", s.strip())
        name, inner = m.group(1), m.group(2).strip().rstrip("]|")
        idx = tuple(int(self.val(t)) for t in inner.split(",") if t.strip())
        return name, idx

    def flat_at(self, name, idx):
        """(flat view of the buffer, flat offset of idx): vector accesses start
        at an element and run along the innermost dimension."""
        a = self.env[name]
        return a.reshape(-1), int(np.ravel_multi_index(idx, a.shape)) if idx else 0

    def stmt(self, s):
        if s.startswith("krnl.store") or s.startswith("memref.store"):
            m = re.match(r"(?:krnl|memref)\.store (%\w+), (.+?) : memref", s)
            name, idx = self.memref_index(m.group(2))
            self.env[name][idx] = self.val(m.group(1))
            return
        if s.startswith("affine.store"):
            m = re.match(r"affine\.store (%\w+), (.+?) : memref", s)
            name, idx = self.memref_index(m.group(2))
            self.env[name][idx] = self.val(m.group(1))
            return
        if s.startswith("vector.store"):
            m = re.match(r"vector\.store (%\w+), (.+?) : memref<[^>]*>, vector<(\d+)x", s)
            name, idx = self.memref_index(m.group(2))
            flat, at = self.flat_at(name, idx)
            flat[at:at + int(m.group(3))] = self.val(m.group(1))
            return
        mb = re.match(r"(%\w+), (%\w+) = krnl\.block (%\w+(?:#\d+)?) (\d+)", s)
        if mb:
            self.blocks[mb.group(1)] = (mb.group(3), int(mb.group(4)))
            return
        if s.startswith("krnl.memset"):
            m = re.match(r"krnl\.memset (%\w+), (%\w+)", s)
            self.env[m.group(1)][...] = self.val(m.group(2))
            return
        m = re.match(r"(%\w+)(?::(\d+))?\s*=\s*(.*)$", s)
        if not m:
            raise ValueError("cannot parse %r" % s)
        dst, nres, rhs = m.group(1), m.group(2), m.group(3)
        op = re.match(r'"?([\w.]+)"?', rhs).group(1)
        if op == "krnl.global":
            g = re.search(r"value = dense<(.+?)> : tensor<((?:\d+x)*)(\w+)>", rhs)
            dims = [int(d) for d in g.group(2).split("x") if d]
            data = np.array(eval(g.group(1), {"__builtins__": {}}), _NP[g.group(3)])
            self.env[dst] = np.broadcast_to(data, dims).copy() if dims else data.reshape(())
            return
        if op == "krnl.define_loops":
            return
        if op.startswith("krnl.get_induction_var_value"):
            loops = [t.strip() for t in re.search(r"\(([^)]*)\)", rhs).group(1).split(",")]
            if nres:
                for k, L in enumerate(loops):
                    self.env["%s#%d" % (dst, k)] = self.loop_iv[L]
            else:
                self.env[dst] = self.loop_iv[loops[0]]
            return
        ty = rhs.rsplit(":", 1)[1].strip() if ":" in rhs else ""
        args = rhs[rhs.index(op) + len(op):].lstrip('"').rsplit(":", 1)[0]
        if op == "arith.constant" and "dense<" in rhs:
            g = re.search(r"dense<(.+?)> : vector<(\d+)xf32>", rhs)
            self.env[dst] = np.full(int(g.group(2)), np.float32(float(g.group(1))), np.float32)
            return
        if op == "arith.constant":
            lit, cty = rhs[rhs.index(op) + len(op):].rsplit(":", 1)
            lit, cty = lit.strip(), cty.strip()
            if cty == "f32":
                if lit.startswith("0x"):
                    self.env[dst] = np.array([int(lit, 16)], np.uint32).view(np.float32)[0]
                else:
                    self.env[dst] = np.float32(float(lit))
            else:
                self.env[dst] = int(lit)
            return
        if op == "memref.alloc":
            mt = re.search(r"memref<((?:[\d?]+x)*)(\w+)>", rhs)
            dims = [d for d in mt.group(1).split("x") if d]
            dyn = [int(self.val(t)) for t in
                   re.search(r"memref\.alloc\(([^)]*)\)", rhs).group(1).split(",") if t.strip()]
            shape = [dyn.pop(0) if d == "?" else int(d) for d in dims]
            self.env[dst] = np.zeros(shape, _NP[mt.group(2)])
            return
        if op == "memref.dim":
            a = [t.strip() for t in args.split(",")]
            self.env[dst] = int(self.env[a[0]].shape[int(self.val(a[1]))])
            return
        if op == "memref.reshape":
            src = re.match(r"\s*(%\w+)", args).group(1)
            to = re.search(r"->\s*memref<((?:\d+x)+)\w+>\s*$", rhs)
            shape = [int(d) for d in to.group(1).split("x") if d] if to else [-1]
            self.env[dst] = self.env[src].reshape(shape)   # a view of the same buffer
            return
        if op == "memref.reinterpret_cast":
            src = re.match(r"\s*(%\w+)", args).group(1)
            sizes = [int(t) for t in re.search(r"sizes: \[([^\]]*)\]", rhs).group(1).split(",")]
            self.env[dst] = self.env[src].reshape(sizes)  # dense strides in these tests
            return
        if op == "affine.apply":
            m2 = re.match(r"\s*(%\w+)\((.*?)\)(?:\|(.*?)\|)?", args)
            dims = [self.val(t) for t in m2.group(2).split(",") if t.strip()]
            syms = [self.val(t) for t in (m2.group(3) or "").split(",") if t.strip()]
            self.env[dst] = self.apply_map(m2.group(1), dims, syms)
            return
        if op == "vector.load":
            m2 = re.match(r"(.+?) : memref<[^>]*>, vector<(\d+)x", rhs[rhs.index(op) + len(op):])
            name, idx = self.memref_index(m2.group(1).strip())
            flat, at = self.flat_at(name, idx)
            self.env[dst] = flat[at:at + int(m2.group(2))].copy()
            return
        if op == "vector.shuffle":
            m2 = re.match(r"\s*(%\w+), (%\w+) \[([\d, ]+)\]", rhs[rhs.index(op) + len(op):])
            both = np.concatenate([self.val(m2.group(1)), self.val(m2.group(2))])
            self.env[dst] = both[[int(t) for t in m2.group(3).split(",")]].astype(np.float32)
            return
        if op == "vector.broadcast":
            m2 = re.match(r"\s*(%\w+) : f32 to vector<(\d+)xf32>", rhs[rhs.index(op) + len(op):])
            self.env[dst] = np.full(int(m2.group(2)), np.float32(self.val(m2.group(1))), np.float32)
            return
        if op in ("krnl.load", "memref.load"):
            name, idx = self.memref_index(args.strip())
            v = self.env[name][idx]
            self.env[dst] = np.float32(v) if self.env[name].dtype == np.float32 else int(v)
            return
        a = [t.strip() for t in args.split(",")]
        f32 = np.float32
        if op in ("arith.addf", "arith.subf", "arith.mulf", "arith.divf"):
            x, y = f32(self.val(a[0])), f32(self.val(a[1]))
            with np.errstate(all="ignore"):
                self.env[dst] = {"arith.addf": x + y, "arith.subf": x - y,
                                 "arith.mulf": x * y, "arith.divf": x / y}[op]
        elif op == "arith.minnumf" or op == "arith.maxnumf":
            x, y = f32(self.val(a[0])), f32(self.val(a[1]))
            fn = np.fmin if op.endswith("minnumf") else np.fmax   # NaN-ignoring
            self.env[dst] = f32(fn(x, y))
        elif op == "math.exp":
            self.env[dst] = _libm_map(_libm.expf, f32(self.val(a[0])))
        elif op == "math.erf":
            self.env[dst] = _libm_map(_libm.erff, f32(self.val(a[0])))
        elif op == "math.sqrt":
            self.env[dst] = f32(np.sqrt(f32(self.val(a[0]))))
        elif op == "math.floor":
            self.env[dst] = f32(np.floor(f32(self.val(a[0]))))
        elif op == "arith.cmpf":
            pred = a[0]
            x, y = f32(self.val(a[1])), f32(self.val(a[2]))
            self.env[dst] = {"ogt": x > y, "oeq": x == y, "olt": x < y,
                             "oge": x >= y, "ole": x <= y}[pred]
        elif op == "arith.select":
            self.env[dst] = self.val(a[1]) if self.val(a[0]) else self.val(a[2])
        elif op in ("arith.addi", "arith.subi", "arith.muli"):
            x, y = int(self.val(a[0])), int(self.val(a[1]))
            r = {"arith.addi": x + y, "arith.subi": x - y, "arith.muli": x * y}[op]
            self.env[dst] = self.wrap(r, ty)
        elif op in ("arith.extsi", "arith.extui", "arith.trunci"):
            src_ty, dst_ty = [t.strip() for t in ty.split(" to ")]
            x = int(self.val(a[0]))
            if op == "arith.extui":
                x &= (1 << {"i8": 8, "i16": 16, "i32": 32}[src_ty]) - 1
            self.env[dst] = self.wrap(x, dst_ty)
        elif op in ("arith.sitofp", "arith.uitofp"):
            src_ty = ty.split(" to ")[0].strip()
            x = int(self.val(a[0]))
            if op == "arith.uitofp":
                x &= (1 << {"i8": 8, "i16": 16, "i32": 32}[src_ty]) - 1
            self.env[dst] = f32(x)
        elif op in ("arith.fptosi", "arith.fptoui"):
            dst_ty = ty.split(" to ")[1].strip()
            x = f32(self.val(a[0]))
            if not np.isfinite(x):
                raise ValueError("fp to int of a non-finite value (poison in LLVM)")
            self.env[dst] = self.wrap(int(np.trunc(x)), dst_ty)
        elif op == "builtin.unrealized_conversion_cast":
            src_ty, dst_ty = [t.strip() for t in ty.split(" to ")]
            x = self.val(a[0])
            self.env[dst] = self.wrap(x, dst_ty) if dst_ty in ("i8", "ui8", "i16", "i32") else x
        else:
            raise NotImplementedError(op + " in: " + s)


def run_lit_function(stmts, params, maps=None, param_names=None):
    it = Interp(stmts, maps)
    names = it.run(params, param_names)
    return it, names
