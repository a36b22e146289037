"""kaon_b200 — the fused optimizer step of kaon (Koronos/K-Optimizers) on NVIDIA B200.

Drop-in for the reference's ``kaon`` classes on the fused-step path: same constructors, param-group keys,
``state_dict`` layout and errors; the step itself runs as hand-written sm_100a CUDA kernels reached
through a C ABI (``libkaon_b200.so``, declared in ``include/kaon_b200.h``).  CUDA tensors only.
"""
from ._version import __version__
from .adakaon import Adakaon
from .adamuon import AdaMuon
from .adapnm import AdaPNM
from .kprodigy import KProdigy
from .lion import Lion
from .nekaon import Nekaon

__all__ = ["AdaMuon", "AdaPNM", "Adakaon", "KProdigy", "Lion", "Nekaon", "__version__"]
