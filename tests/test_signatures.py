"""The ctypes argument lists agree with the C declarations they call.

A list with two arguments swapped still loads and still runs; a pointer
passed where the C side reads an int loses half its bits. So the exported
declarations are read from the sources as text and compared, argument by
argument, with the table the loader gives to ctypes.
"""
import re
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

from dynalm_b200.kernels import ops

CSRC = Path(ops.__file__).resolve().parent.parent / "csrc"
DECLARATION = re.compile(r"DL_EXPORT\s+[\w\s\*]+?\b(dl_\w+)\s*\(([^)]*)\)\s*\{")


def argument_kind(text):
    if "*" in text or "cudaStream_t" in text:
        return c_void_p
    if re.match(r"(const\s+)?float\b", text):
        return c_float
    if re.match(r"(const\s+)?long long\b", text):
        return c_longlong
    if re.match(r"(const\s+)?(unsigned\s+)?int\b", text):
        return c_int
    raise AssertionError(f"an argument of a kind the table has no name for: {text!r}")


def declarations():
    found = {}
    for path in sorted(CSRC.iterdir()):
        if path.suffix not in (".cu", ".cuh", ".h"):
            continue
        for match in DECLARATION.finditer(path.read_text()):
            name, args = match.group(1), match.group(2)
            found[name] = [argument_kind(a.strip()) for a in args.split(",") if a.strip()]
    return found


def test_every_signature_matches_its_declaration():
    declared = declarations()
    checked = 0
    for library, table in ops._SIGNATURES.items():
        for name, signature in table.items():
            assert name in declared, f"{library}: {name} is in the table but no source exports it"
            assert list(signature) == declared[name], (
                f"{name}: the table has {len(signature)} arguments "
                f"{[k.__name__ for k in signature]}, the source {len(declared[name])} "
                f"{[k.__name__ for k in declared[name]]}")
            checked += 1
    assert checked >= 20


def test_every_export_of_a_loaded_source_is_in_the_table():
    declared = declarations()
    listed = {name for table in ops._SIGNATURES.values() for name in table}
    elsewhere = {
        # The checked build's two calls get their argument lists where they are looked up, once per library.
        "dl_check_limits", "dl_check_take",
        # Sizes asked of the C side by tests and by C programs; they launch nothing.
        "dl_paged_attention_decode_tile", "dl_paged_attention_decode_scratch", "dl_gemm_skinny_argmax_blocks",
        # The allocation-free entry point and its messages are called by C programs, not through this table.
        "dl_paged_attention_decode_noalloc", "dl_noalloc_strerror",
    }
    missing = {n for n in declared if n not in listed} - elsewhere
    assert not missing, f"exported but without a signature: {sorted(missing)}"
