"""The Zig side of the drop-in (zig/src/) is kept as source: no Zig toolchain exists where this repository is
built.  What can be checked without one is the boundary: every launcher triple and every `mp*` utility the Zig files
call must be declared in include/*.h, with the number of arguments the Zig call passes."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
ZIG = sorted((ROOT / "zig" / "src").rglob("*.zig"))


def split_top_level(text: str):
    """Comma-separated items of `text`, ignoring commas nested in (), {} or []."""
    items, depth, cur = [], 0, ""
    for ch in text:
        if ch in "({[":
            depth += 1
        elif ch in ")}]":
            depth -= 1
        if ch == "," and depth == 0:
            items.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        items.append(cur)
    return [i.strip() for i in items if i.strip()]


def balanced(text: str, start: int, open_ch: str, close_ch: str) -> str:
    """Contents of the bracket that opens at text[start]."""
    assert text[start] == open_ch
    depth = 0
    for i in range(start, len(text)):
        if text[i] == open_ch:
            depth += 1
        elif text[i] == close_ch:
            depth -= 1
            if depth == 0:
                return text[start + 1:i]
    raise AssertionError("unbalanced bracket")


def header_arities():
    """name -> number of parameters, for MP_DECL3 triples (keyed without suffix) and MP_EXTERN_C functions."""
    triples, functions = {}, {}
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        for m in re.finditer(r"^MP_DECL3\(", text, flags=re.M):   # (declarations, not the macro's own #define)
            body = split_top_level(balanced(text, m.end() - 1, "(", ")"))
            triples[body[0]] = len(body) - 1
        for m in re.finditer(r"MP_EXTERN_C\s+[\w\s\*]+?\b(\w+)\(", text):
            params = balanced(text, m.end() - 1, "(", ")").strip()
            functions[m.group(1)] = 0 if params in ("", "void") else len(split_top_level(params))
    return triples, functions


def strip_comments(src: str) -> str:
    return re.sub(r"//[^\n]*", "", src)


def test_zig_sources_exist():
    names = {p.name for p in ZIG}
    for want in ("kernels.zig", "cimport.zig", "gradients.zig", "selu.zig", "linear.zig", "softmax.zig", "rmsnorm.zig", "ssd.zig",
                 "permutate.zig", "contraction.zig", "optimizer.zig", "metaphor_additions.zig"):
        assert want in names, want
    assert (ROOT / "oracle" / "zig" / "oracle.zig").exists()


def test_kernel_arrays_name_only_declared_launchers():
    triples, _ = header_arities()
    text = strip_comments((ROOT / "zig" / "src" / "core" / "kernels.zig").read_text())
    arrays = re.findall(r"pub const (\w+) = dispatch_array", text)
    assert len(arrays) >= 50
    for name in arrays:
        assert name in triples, f"kernels.zig names launch_{name}_*, which include/mp_kernels.h does not declare"
    for sym in re.findall(r"decls\.(launch_\w+)", text):
        base, sfx = sym[len("launch_"):].rsplit("_", 1)
        assert sfx in ("r16", "r32", "r64") and base in triples, sym
    # the twenty launchers of the reference must all be there (src/cuda/kernel_decls.h)
    # ... and every triple the headers declare has its array
    for name in triples:
        assert name in arrays, f"include/mp_kernels.h declares launch_{name}_*, kernels.zig has no array for it"
    for ref in ("reduce_ij_i", "reduce_ij_j", "broadcast_i_ij", "dilate_reverse", "subtraction", "relu_reverse", "dilate", "translate",
                "permutate_ij_ji", "negate", "hadamard_reverse", "inner_product_ij_jk_ik", "hadamard", "fill", "relu", "addition",
                "broadcast_j_ij", "copy", "sequence", "stepwise"):
        assert ref in arrays, ref


def test_every_call_matches_a_declaration_and_its_arity():
    triples, functions = header_arities()
    checked = 0
    for path in ZIG:
        src = strip_comments(path.read_text())
        for m in re.finditer(r"core\.invoke\(core\.kernels\.(\w+),", src):
            name = m.group(1)
            assert name in triples, f"{path.name}: core.kernels.{name} has no MP_DECL3 declaration"
            tuple_start = src.index(".{", m.end())
            args = split_top_level(balanced(src, tuple_start + 1, "{", "}"))
            assert len(args) == triples[name], f"{path.name}: {name} called with {len(args)} arguments, declared with {triples[name]}"
            checked += 1
        for m in re.finditer(r"\bC\.(mp\w+|launch_\w+)\(", src):
            name = m.group(1)
            assert name in functions, f"{path.name}: C.{name} is not declared in include/*.h"
            args = split_top_level(balanced(src, m.end() - 1, "(", ")"))
            assert len(args) == functions[name], f"{path.name}: {name} called with {len(args)} arguments, declared with {functions[name]}"
            checked += 1
    assert checked >= 25
