"""The Rust shim (rust/tkv-sys, rust/tkv-workers) cannot be compiled where it is written, so it is checked
mechanically against include/tkv.h: the generated FFI file is what the generator produces from the current header;
every extern "C" function has the header's name, argument count and argument / return types; every #[repr(C)]
struct has the header's fields in the header's order (and the same size as the ctypes mirror, whose sizes the
C compiler confirms in test_abi_symbols.py); build.rs compiles exactly the sources the Python build compiles;
and every tkv_sys call in the worker crate exists with the number of arguments it is given."""
import ctypes as C
import importlib.util
import os
import re

from tempura_b200 import _build, _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SYS = os.path.join(ROOT, "rust", "tkv-sys")
LIB_RS = os.path.join(SYS, "src", "lib.rs")
WORKERS_RS = os.path.join(ROOT, "rust", "tkv-workers", "src", "lib.rs")


def _gen():
    spec = importlib.util.spec_from_file_location("gen_bindings", os.path.join(SYS, "gen_bindings.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_committed_bindings_are_what_the_generator_makes_of_the_header():
    gen = _gen()
    with open(os.path.join(ROOT, "include", "tkv.h")) as f:
        assert open(LIB_RS).read() == gen.render(f.read()), "run python rust/tkv-sys/gen_bindings.py"


# ---- an independent reading of both files -------------------------------------------------------------------
_C2R = {"int32_t": "i32", "uint32_t": "u32", "uint64_t": "u64", "uint8_t": "u8", "size_t": "usize", "float": "f32",
        "char": "c_char", "void": "c_void"}


def _c_functions():
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "tkv.h")).read(), flags=re.S)
    text = re.sub(r"typedef\s+struct\s+\w+\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)                       # preprocessor lines
    out = {}
    for m in re.finditer(r"(\w[\w\s\*]*?)\b(tkv_\w+)\s*\(([^)]*)\)\s*;", text, flags=re.S):
        args = " ".join(m.group(3).split())
        out[m.group(2)] = ([] if args in ("", "void") else [a.strip() for a in args.split(",")], " ".join(m.group(1).split()))
    return out


def _c_to_rust(decl: str) -> str:
    """`const uint32_t* seq_lens` / `tkv_plan** out` / `uint8_t handle[64]` -> the Rust type a binding must use."""
    d = decl.strip()
    levels = d.count("*") + (1 if re.search(r"\[\d*\]\s*$", d) else 0)
    d = re.sub(r"\[\d*\]\s*$", "", d).replace("*", " ")
    words = d.split()
    const = words[0] == "const"
    base = words[1] if const else words[0]
    r = _C2R.get(base, base)
    for i in range(levels):
        r = ("*const " if const and i == 0 else "*mut ") + r
    return r


def _rust_functions():
    text = open(LIB_RS).read()
    block = text[text.index('extern "C" {'):]
    out = {}
    for m in re.finditer(r"pub fn (tkv_\w+)\((.*?)\)(?:\s*->\s*([^;]+))?;", block):
        params = [p.split(":", 1)[1].strip() for p in m.group(2).split(", ")] if m.group(2).strip() else []
        out[m.group(1)] = (params, (m.group(3) or "").strip())
    return out


def test_every_function_matches_the_header():
    cf, rf = _c_functions(), _rust_functions()
    assert sorted(cf) == sorted(rf) == sorted(_native.SIGNATURES)
    for name, (cargs, cret) in cf.items():
        rargs, rret = rf[name]
        assert len(cargs) == len(rargs), name
        for ca, ra in zip(cargs, rargs):
            assert _c_to_rust(ca) == ra, (name, ca, ra)
        assert (rret == "") == (cret == "void"), name
        if cret != "void":
            assert _c_to_rust(cret + " x") == rret, (name, cret, rret)


def test_every_struct_has_the_headers_fields_in_order_and_the_ctypes_size():
    header = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "tkv.h")).read(), flags=re.S)
    rust = open(LIB_RS).read()
    n = 0
    size = {"i32": 4, "u32": 4, "f32": 4, "u64": 8, "usize": 8, "u8": 1}
    for m in re.finditer(r"typedef\s+struct\s+\w+\s*\{(.*?)\}\s*(\w+)\s*;", header, flags=re.S):
        name = m.group(2)
        c_fields = []
        for decl in m.group(1).split(";"):
            decl = " ".join(decl.split())
            if decl:
                head = re.match(r"^((?:const\s+)?\w+)", decl).group(1)
                for part in decl[len(head):].split(","):
                    c_fields.append((part.replace("*", "").strip(), _c_to_rust(head + part)))
        rs = re.search(r"#\[repr\(C\)\]\s*#\[derive\([^)]*\)\]\s*pub struct " + name + r" \{(.*?)\n\}", rust, flags=re.S)
        assert rs, f"{name} missing or not #[repr(C)]"
        r_fields = [tuple(x.strip() for x in ln.strip().rstrip(",")[4:].split(":", 1)) for ln in rs.group(1).strip().splitlines()]
        assert r_fields == c_fields, name
        # natural alignment: the size follows from the field list; it must be the ctypes mirror's (= the C compiler's)
        def size_align(t):
            if t.startswith("*"):
                return 8, 8
            if t in size:
                return size[t], size[t]
            return C.sizeof(getattr(_native, t)), C.alignment(getattr(_native, t))     # a nested struct (TkvShard in TkvPairing)
        off, align = 0, 1
        for _, t in r_fields:
            sz, al = size_align(t)
            off = (off + al - 1) // al * al + sz
            align = max(align, al)
        off = (off + align - 1) // align * align
        assert off == C.sizeof(getattr(_native, name)), name
        n += 1
    assert n >= 15


def test_build_rs_compiles_the_sources_the_python_build_compiles():
    text = open(os.path.join(SYS, "build.rs")).read()
    listed = re.findall(r'"(tkv_\w+\.(?:cu|cpp))"', text[text.index("const SOURCES"):text.index("];")])
    assert listed == list(_build.SOURCES)
    for flag in ("arch=compute_100a,code=sm_100a", "-fmad=false", "-prec-div=true"):
        assert flag in text and flag in _build.NVCC_FLAGS


def test_worker_crate_calls_exist_with_the_right_arity():
    rf = _rust_functions()
    text = re.sub(r"//.*", "", open(WORKERS_RS).read())
    calls = re.findall(r"\b(tkv_[a-z0-9_]+)\(", text)
    assert {"tkv_init", "tkv_plan_create", "tkv_handoff_enqueue", "tkv_flag_wait_host", "tkv_plan_destroy", "tkv_last_error"} <= set(calls)
    for m in re.finditer(r"\b(tkv_[a-z0-9_]+)\(", text):
        name = m.group(1)
        assert name in rf, name
        depth, i, args, cur = 1, m.end(), [], ""
        while depth:                                   # split the call's arguments at top-level commas
            ch = text[i]
            depth += ch in "([{"
            depth -= ch in ")]}"
            if depth == 1 and ch == ",":
                args.append(cur)
                cur = ""
            elif depth:
                cur += ch
            i += 1
        if cur.strip():
            args.append(cur)
        assert len(args) == len(rf[name][0]), (name, args)
    # the traits implemented are the reference's own
    assert "impl<E: PrefillEngine> PrefillWorker for GpuPrefillWorker<E>" in text
    assert "impl<D: DecodeEngine> DecodeWorker for GpuDecodeWorker<D>" in text
    assert "KernelError::DimensionMismatch { expected, got }" in text and "KernelError::InvalidConfig" in text


def test_the_integration_guide_quotes_the_crates_verbatim():
    """Every fenced rust block of the guide is an excerpt of a file under rust/: the guide cannot drift from the crates."""
    import re
    guide = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```rust\n(.*?)```", guide, flags=re.S)
    assert blocks, "the guide quotes at least the status mapping"
    sources = []
    for dirpath, _, files in os.walk(os.path.join(ROOT, "rust")):
        sources += [open(os.path.join(dirpath, f)).read() for f in files if f.endswith(".rs")]
    for b in blocks:
        assert any(b in src for src in sources), b[:80]
