"""B200-native D-NPEFF factorization engine (drop-in for ``run_nmf_on_pefs``).

The compute lives in ``libdnpeff.so`` (hand-written sm_100a CUDA behind the C
ABI of ``include/dnpeff.h``); this package is a thin ctypes host layer that
mirrors the reference's ``MuNmf`` interface.  There is no CPU fallback: if the
library is missing or no CUDA device answers, calls raise.
"""
from ._lib import DnpeffError, lib, lib_path  # noqa: F401
from .engine import MuNmf, MuNmfParams, preprocess_and_split  # noqa: F401
