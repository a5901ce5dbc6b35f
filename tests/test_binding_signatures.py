"""Every binding of the C ABI agrees with include/b200wmma.h argument for argument: the ctypes table the
tests and the bench call through (cudanative.jl_b200/_lib.py) and the `ccall`s of the Julia wrapper
(cudanative.jl_b200/julia/B200WMMA.jl, which cannot be executed here: Julia is not installed).  A wrong
arity or width in either would pass garbage to a kernel launch without any error."""
import ctypes as C
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200wmma.h"
JULIA = ROOT / "cudanative.jl_b200" / "julia" / "B200WMMA.jl"

# C type -> class: i32, i64, u32, u64, f32, size, ptr
def c_class(ctype: str) -> str:
    t = " ".join(ctype.replace("const", " ").split())
    if "*" in t or t in ("b200_stream",):
        return "ptr"
    return {"int": "i32", "int64_t": "i64", "uint32_t": "u32", "uint64_t": "u64", "float": "f32", "size_t": "size",
            "void": "void"}[t]


def header_prototypes() -> dict:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    protos = {}
    for ret, name, args in re.findall(r"([A-Za-z_][A-Za-z0-9_ \*]*?)\s*\b(b200_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        params = []
        args = args.strip()
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                m = re.match(r"(.*?)([A-Za-z_][A-Za-z0-9_]*)$", a)  # strip the parameter name
                params.append(c_class(m.group(1).strip()))
        protos[name] = (c_class(ret.strip()) if "*" not in ret else "ptr", params)
    return protos


def test_header_parses_completely():
    protos = header_prototypes()
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    assert sorted(protos) == sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))
    assert protos["b200_gemm_f16f32"] == ("i32", ["ptr", "ptr", "i32", "i32", "i64", "i64", "i64", "f32", "ptr", "i64", "ptr",
                                                  "i64", "f32", "ptr", "i64", "ptr", "i64"])
    assert protos["b200_last_error"] == ("ptr", [])


def ctypes_class(t) -> str:
    if t is None:
        return "void"
    if t in (C.c_void_p, C.c_char_p) or isinstance(t, type(C.POINTER(C.c_int))) and issubclass(t, C._Pointer):
        return "ptr"
    return {C.c_int: "i32", C.c_int64: "i64", C.c_uint32: "u32", C.c_uint64: "u64", C.c_float: "f32", C.c_size_t: "size"}[t]


def test_ctypes_table_matches_the_header(pkg):
    protos = header_prototypes()
    for name, (restype, argtypes) in pkg._lib.SIGNATURES.items():
        want_ret, want_args = protos[name]
        got_args = [ctypes_class(t) for t in argtypes]
        # size_t and uint64_t are the same width on every platform this library targets (LP64)
        norm = lambda xs: ["u64" if x == "size" else x for x in xs]  # noqa: E731
        assert norm(got_args) == norm(want_args), f"{name}: ctypes {got_args} vs header {want_args}"
        assert ctypes_class(restype) == want_ret, f"{name}: return type"


JULIA_CLASS = {"Cint": "i32", "Int64": "i64", "UInt32": "u32", "UInt64": "u64", "Cfloat": "f32", "Csize_t": "size",
               "Cstring": "ptr", "Cvoid": "void"}


def julia_class(t: str) -> str:
    t = t.strip()
    if t.startswith(("Ptr{", "CuPtr{", "Ref{")):
        return "ptr"
    return JULIA_CLASS[t]


def split_top_level(s: str) -> list:
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch in "({[":
            depth += 1
        elif ch in ")}]":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur)
    return out


def julia_ccalls() -> list:
    """(name, return class, argument classes, number of values passed) of every ccall in the wrapper."""
    src = re.sub(r"#=.*?=#", "", JULIA.read_text(), flags=re.S)
    src = "\n".join(line.split("#")[0] if not line.lstrip().startswith("#") else "" for line in src.splitlines())
    calls = []
    for m in re.finditer(r"ccall\(\(:(b200_[a-z0-9_]+), lib\),", src):
        # take the balanced argument list of this ccall
        start = src.index("(", m.start())
        depth, i = 0, start
        while True:
            depth += src[i] == "("
            depth -= src[i] == ")"
            if depth == 0:
                break
            i += 1
        parts = split_top_level(src[start + 1:i])
        ret = julia_class(parts[1])
        types = parts[2].strip()
        assert types.startswith("(") and types.endswith(")")
        arg_types = [julia_class(t) for t in split_top_level(types[1:-1]) if t.strip()]
        calls.append((m.group(1), ret, arg_types, len(parts) - 3))
    return calls


def test_julia_ccalls_match_the_header():
    protos = header_prototypes()
    calls = julia_ccalls()
    assert len(calls) >= 28
    seen = set()
    for name, ret, arg_types, n_values in calls:
        want_ret, want_args = protos[name]
        assert arg_types == want_args, f"{name}: Julia {arg_types} vs header {want_args}"
        assert ret == want_ret, f"{name}: return type {ret} vs {want_ret}"
        assert n_values == len(want_args), f"{name}: {n_values} values passed for {len(want_args)} parameters"
        seen.add(name)
    # the entry points of the path must all be bound
    for must in ("b200_create", "b200_destroy", "b200_gemm_f16f32", "b200_gemm_f16f32_host", "b200_gemm_strided_batched",
                 "b200_wmma_load", "b200_wmma_fill_c", "b200_wmma_mma", "b200_wmma_store_d", "b200_wmma_bcast",
                 "b200_wmma_16x16x16", "b200_last_error", "b200_malloc", "b200_free", "b200_set_option", "b200_device_status",
                 "b200_gemm_f16_typed", "b200_gemm_f16f32_gated", "b200_gemm_f16f32_splitk_static", "b200_static_status",
                 "b200_static_warmup", "b200_sharded_create", "b200_sharded_info", "b200_sharded_ipc_blob",
                 "b200_sharded_attach", "b200_sharded_run", "b200_sharded_wait", "b200_sharded_destroy"):
        assert must in seen, f"{must} has no ccall in B200WMMA.jl"
