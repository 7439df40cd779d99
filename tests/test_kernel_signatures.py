"""The table of argument types that the Python side gives ctypes must agree with the C declarations:
a wrong letter there would hand a kernel a truncated pointer.  The declarations are read from the
sources as text; nothing is compiled."""
import glob
import os
import re

from idempotent_llm_b200.kernels import ops

CSRC = os.path.join(os.path.dirname(ops.__file__), "..", "csrc")


def _declared():
    found = {}
    for path in sorted(glob.glob(os.path.join(CSRC, "*.cu"))):
        text = open(path).read()
        for m in re.finditer(r'extern "C" ([\w ]+?\*?) ?(idm_\w+)\(([^)]*)\)', text):
            letters = ""
            for arg in (a.strip() for a in m.group(3).replace("\n", " ").split(",")):
                if not arg:
                    continue
                if "*" in arg or arg.startswith("cudaStream_t"):
                    letters += "p"
                elif arg.startswith("long long"):
                    letters += "q"
                elif arg.startswith("float"):
                    letters += "f"
                elif arg.startswith("int"):
                    letters += "i"
                else:
                    raise AssertionError(f"{m.group(2)}: argument {arg!r} has a type the table has no letter for")
            found[m.group(2)] = (m.group(1).strip(), letters)
    return found


def test_every_entry_point_is_in_the_table_with_the_declared_types():
    declared = _declared()
    assert set(declared) == set(ops.SIGNATURES), (
        f"only declared: {sorted(set(declared) - set(ops.SIGNATURES))}; "
        f"only in the table: {sorted(set(ops.SIGNATURES) - set(declared))}")
    results = {"int": ops.c_int, "long long": ops.c_longlong, "void": None, "const char*": ops.ctypes.c_char_p}
    for name, (result, letters) in declared.items():
        want_result, want_letters = ops.SIGNATURES[name]
        assert letters == want_letters, f"{name}: declared {letters}, table {want_letters}"
        assert results[result] is want_result, f"{name}: returns {result}"
