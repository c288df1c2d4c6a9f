"""The C-ABI shared library loads and exports every symbol declared in include/*.h (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names += re.findall(r"SB_API\s+[\w\s\*]+?\b(sb_\w+)\s*\(", text)
    return names


@pytest.fixture(scope="module")
def kernel_lib():
    from torch_supa_b200 import _build, capi

    _build.build_kernels()
    return ctypes.CDLL(str(capi.LIB_PATH))


def test_header_declares_the_hot_path():
    names = declared_symbols()
    for required in ("sb_ce_forward_backward", "sb_ce_count_valid", "sb_elementwise", "sb_reduce",
                     "sb_log_softmax_forward", "sb_nll_loss_forward"):
        assert required in names


def test_every_declared_symbol_is_exported(kernel_lib):
    missing = [n for n in declared_symbols() if not hasattr(kernel_lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_identification_calls(kernel_lib):
    kernel_lib.sb_version.restype = ctypes.c_char_p
    assert b"sm_100a" in kernel_lib.sb_version()
    assert kernel_lib.sb_built_for_sm() == 100
    kernel_lib.sb_dtype_size.restype = ctypes.c_size_t
    assert [kernel_lib.sb_dtype_size(i) for i in range(10)] == [1, 1, 1, 2, 4, 8, 2, 2, 4, 8]
    kernel_lib.sb_status_string.restype = ctypes.c_char_p
    assert kernel_lib.sb_status_string(-1) == b"invalid argument"


def test_argument_validation_needs_no_gpu(kernel_lib):
    """Launchers reject bad descriptors before touching the device."""
    from torch_supa_b200 import capi

    args = capi.CEArgs()
    args.rows, args.classes = -1, 10
    assert kernel_lib.sb_ce_forward_backward(ctypes.byref(args), None) == -1
    desc = capi.EWDesc()
    desc.op, desc.ndim, desc.noperands = 99, 1, 2
    assert kernel_lib.sb_elementwise(ctypes.byref(desc), None) == -1
    assert kernel_lib.sb_elementwise(None, None) == -1
    rdesc = capi.ReduceDesc()
    rdesc.op, rdesc.ndim = 0, 0
    assert kernel_lib.sb_reduce(ctypes.byref(rdesc), None) == -1
    rng = capi.RngArgs()
    rng.dst, rng.dtype, rng.kind, rng.numel, rng.a, rng.b, rng.offset = 0x1000, 8, capi.SB_RNG_UNIFORM, 16, 0.0, 1.0, 2
    assert kernel_lib.sb_rng_fill(ctypes.byref(rng), None) == -1          # an offset that is not a whole Philox block
    rng.offset, rng.a, rng.b = 4, 1.0, 0.0
    assert kernel_lib.sb_rng_fill(ctypes.byref(rng), None) == -1          # from > to
    rng.a, rng.b, rng.dtype = 0.0, 1.0, 4
    assert kernel_lib.sb_rng_fill(ctypes.byref(rng), None) < 0            # uniform into int32
    rng.numel = 0
    assert kernel_lib.sb_rng_fill(ctypes.byref(rng), None) == 0           # nothing to do
    assert kernel_lib.sb_dropout(ctypes.c_void_p(0x1000), ctypes.c_void_p(0x2000), ctypes.c_void_p(0x3000), 8, ctypes.c_int64(16),
                                 ctypes.c_double(1.5), ctypes.c_uint64(1), ctypes.c_uint64(0), None) == -1


def test_path_classifier_runs_on_host(kernel_lib):
    """The elementwise classifier is pure host code: the benchmark shapes map to the intended paths."""
    from torch_supa_b200 import capi

    def desc(op, sizes, strides, dtypes, common):
        d = capi.EWDesc()
        d.op, d.ndim, d.noperands, d.common_dtype = op, len(sizes), len(strides), common
        for i, s in enumerate(sizes):
            d.sizes[i] = s
        for k, st in enumerate(strides):
            for i, s in enumerate(st):
                d.strides[k][i] = s
            d.data[k] = 0x1000 * (k + 1)
            d.dtype[k] = dtypes[k]
        return d

    F16, BF16, F32, I32 = capi.F16, capi.BF16, capi.F32, capi.I32
    contiguous = desc(capi.EW_ADD, [1 << 20], [[1], [1], [1]], [F32, I32, F32], F32)
    assert kernel_lib.sb_elementwise_path(ctypes.byref(contiguous)) == 0
    broadcast = desc(capi.EW_ADD, [4096, 2048, 64], [[1, 4096, 8388608], [1, 0, 4096], [1, 4096, 0]], [F16] * 3, F16)
    assert kernel_lib.sb_elementwise_path(ctypes.byref(broadcast)) == 1
    halves = desc(capi.EW_SILU, [11008, 16384], [[1, 11008], [1, 22016]], [BF16] * 2, BF16)
    assert kernel_lib.sb_elementwise_path(ctypes.byref(halves)) == 1
    transposed = desc(capi.EW_MUL, [4096, 8192], [[1, 4096], [1, 4096], [8192, 1]], [F32] * 3, F32)
    assert kernel_lib.sb_elementwise_path(ctypes.byref(transposed)) == 2
    odd = desc(capi.EW_MUL, [5, 7, 3], [[3, 15, 1], [1, 5, 35], [1, 5, 35]], [F32] * 3, F32)
    assert kernel_lib.sb_elementwise_path(ctypes.byref(odd)) == 3


def test_ctypes_structures_match_the_header(tmp_path):
    """Every descriptor the Python binding passes by pointer has the size and the field offsets the C compiler gives the
    header's struct: a field added to the header but not to the binding makes the library read past the Python buffer."""
    import subprocess

    from torch_supa_b200 import capi

    pairs = {"sb_ce_args": capi.CEArgs, "sb_xchg": capi.Xchg, "sb_ce_prob_args": capi.CEProbArgs, "sb_rng_args": capi.RngArgs,
             "sb_nll_args": capi.NLLArgs, "sb_nll_nd_args": capi.NLLNdArgs, "sb_ew_desc": capi.EWDesc, "sb_reduce_desc": capi.ReduceDesc}
    header = (ROOT / "include" / "supa_b200_kernels.h").read_text()
    assert set(re.findall(r"typedef struct (sb_\w+) \{", header)) == set(pairs), "a struct of the header has no ctypes mirror (or the reverse)"
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "supa_b200_kernels.h"', "int main(void) {"]
    for name, cls in pairs.items():
        lines.append(f'  printf("{name} size %zu\\n", sizeof({name}));')
        body = header[header.index(f"typedef struct {name} {{"):header.index(f"}} {name};")]
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        c_fields = []
        for statement in body.split("{", 1)[1].split(";"):
            for declarator in statement.split(","):
                m = re.search(r"(\w+)\s*(?:\[[^\]]*\])*\s*$", declarator.strip())
                if m:
                    c_fields.append(m.group(1))
        py_fields = [f[0] for f in cls._fields_]
        assert len(c_fields) == len(py_fields), f"{name}: {c_fields} vs {py_fields}"
        for c_name in c_fields:
            lines.append(f'  printf("{name} {c_name} %zu\\n", offsetof({name}, {c_name}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    got = {}
    for line in out:
        if line:
            name, field, value = line.split()
            got.setdefault(name, []).append((field, int(value)))
    for name, cls in pairs.items():
        assert got[name][0] == ("size", ctypes.sizeof(cls)), name
        offsets = [v for _, v in got[name][1:]]
        assert offsets == [getattr(cls, f[0]).offset for f in cls._fields_], f"{name}: field offsets differ"
