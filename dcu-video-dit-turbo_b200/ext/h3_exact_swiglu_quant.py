"""Stand-in for the reference's compiled extension module `h3_exact_swiglu_quant`
(kernels/swiglu-quant/swiglu_quant.cpp:5-9 in the reference): same module name, same callables, backed by libb2dit.so.

Load it the way the reference's launcher loads its DSO, by file path:
    spec = importlib.util.spec_from_file_location("h3_exact_swiglu_quant", "<this file>")
so pointing the launcher's *_SO environment variable at this file is the whole
integration.  Importing it loads the CUDA library and raises if that is missing."""
import importlib.util as _u
from pathlib import Path as _P

_spec = _u.spec_from_file_location("_b2dit_ext_bootstrap", _P(__file__).with_name("_bootstrap.py"))
_boot = _u.module_from_spec(_spec)
_spec.loader.exec_module(_boot)
_pkg = _boot.package()
_pkg._lib.load()

swiglu_quantize_int8_rowwise = _pkg.ops.swiglu_quantize_int8_rowwise
