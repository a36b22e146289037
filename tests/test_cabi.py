"""The C-ABI library loads and exports every symbol that include/kaon_b200.h declares; the host-side
argument checks answer without a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "kaon_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kaon_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared()
    assert "kaon_lion_step" in names and "kaon_plan_create" in names and len(names) >= 12


def test_library_exports_every_declared_symbol():
    from kaon_b200 import _build, _lib
    _build.build()
    lib = _lib.lib()
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, missing
    assert lib.kaon_abi_version() == 2


def test_host_side_argument_checks():
    from kaon_b200 import _lib
    lib = _lib.lib()
    rc = lib.kaon_plan_create(None, 0, 0, 0, None, 0)
    assert rc == -1 and b"null" in lib.kaon_last_error()
    with pytest.raises(_lib.KaonError):
        _lib.check(rc)
    assert lib.kaon_lion_step(None, None, C.c_uint64(0), C.c_uint32(0), None) == -1
    assert lib.kaon_codec_encode_4bit(None, C.c_int64(1), C.c_int64(128), None, None, None) == -1


def test_cpu_tensors_are_refused():
    import torch
    import kaon_b200
    from kaon_b200._lib import KaonError
    p = torch.nn.Parameter(torch.zeros(4, 4))
    opt = kaon_b200.Lion([p], momentum_dtype="4bit")
    p.grad = torch.zeros(4, 4)
    with pytest.raises(KaonError, match="CUDA tensors only"):
        opt.step()


def test_integration_doc_structs_match_the_header():
    """The ctypes structs printed in INTEGRATION.md have the size and field order the library uses."""
    from kaon_b200 import _lib
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    ns = {"C": C}
    for name in ("TensorDesc", "LionHParams", "AdaPNMHParams", "KProdigyPass1", "KProdigyPass2"):
        m = re.search(r"class %s\(C\.Structure\):.*?\n    _fields_ = \[(.*?)\]" % name, text, flags=re.S)
        assert m, name
        exec("class %s(C.Structure):\n    _fields_ = [%s]" % (name, m.group(1)), ns)  # noqa: S102
        doc, ours = ns[name], getattr(_lib, name)
        assert C.sizeof(doc) == C.sizeof(ours), (name, C.sizeof(doc), C.sizeof(ours))
        assert [f[0] for f in doc._fields_] == [f[0] for f in ours._fields_]
    assert C.sizeof(ns["TensorDesc"]) == 80 and C.sizeof(ns["AdaPNMHParams"]) == 80
    assert C.sizeof(ns["KProdigyPass1"]) == 72 and C.sizeof(ns["KProdigyPass2"]) == 48
    assert '"kahan": 2' in text
