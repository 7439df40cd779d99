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


def test_the_records_of_a_step_program_are_the_same_on_both_sides():
    """Array lengths and the numbers of the kinds of call in ``step_program.h`` against ``kernels/program.py``
    (sizes and offsets are compared again with the compiled library when it is loaded)."""
    from idempotent_llm_b200.kernels import program
    text = open(os.path.join(CSRC, "step_program.h")).read()
    defines = {m.group(1): int(m.group(2)) for m in re.finditer(r"#define (IDM_\w+) (\d+)", text)}
    assert defines["IDM_OP_INTS"] == program.OP_INTS
    assert defines["IDM_OP_FLOATS"] == program.OP_FLOATS
    assert defines["IDM_OP_POINTERS"] == program.OP_POINTERS
    assert defines["IDM_PROGRAM_BUFFERS"] == program.MAX_BUFFERS
    assert defines["IDM_PROGRAM_PLANS"] == program.MAX_PLANS
    kinds = {m.group(1): int(m.group(2)) for m in re.finditer(r"IDM_OP_(\w+) = (\d+),", text)}
    assert kinds == {"EMBED": program.EMBED, "ROPE_TABLE": program.ROPE_TABLE, "ADD_RMSNORM": program.ADD_RMSNORM,
                     "GEMM_QKV": program.GEMM_QKV, "ATTENTION": program.ATTENTION,
                     "GEMM_RESIDUAL": program.GEMM_RESIDUAL, "GEMM_SWIGLU": program.GEMM_SWIGLU,
                     "GEMM_STORE": program.GEMM_STORE}
    # every field of the C records appears in the binding's, in the same order
    def fields(struct_name):
        body = re.search(r"struct %s \{(.*?)\};" % struct_name, text, re.S).group(1)
        body = re.sub(r"//[^\n]*", "", body)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            decl = re.sub(r"^(const )?\w+\*? ", "", decl)
            for part in decl.split(","):
                names.append(re.sub(r"[\*\s]|\[.*\]", "", part))
        return names
    assert fields("IdmOp") == [f[0] for f in program.IdmOp._fields_]
    assert fields("IdmAttnPlan") == [f[0] for f in program.IdmAttnPlan._fields_]
    assert fields("IdmStep") == [f[0] for f in program.IdmStep._fields_]
