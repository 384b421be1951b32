"""Makes the aimet_torch reference importable from its source tree (fixture generation only).

The reference imports a few packages that are not installed (bokeh, onnx, onnxruntime, onnxscript,
onnx_ir) at module load although the quantization-simulation path never calls them; they are
replaced by inert stand-ins.  Set AIMET_REFERENCE_ROOT to the checkout of the reference.
"""

import importlib.abc
import importlib.machinery
import os
import sys
from unittest.mock import MagicMock

_STUB_ROOTS = {"bokeh", "onnx", "onnxruntime", "onnxscript", "onnx_ir"}
REFERENCE_ROOT = os.environ.get("AIMET_REFERENCE_ROOT", "")


class _Loader(importlib.abc.Loader):
    def create_module(self, spec):
        m = MagicMock(name=spec.name)
        m.__name__, m.__path__, m.__spec__, m.__version__ = spec.name, [], spec, "1.18.0"
        return m

    def exec_module(self, module):
        pass


class _Finder(importlib.abc.MetaPathFinder):
    def find_spec(self, name, path, target=None):
        if name.split(".")[0] in _STUB_ROOTS:
            return importlib.machinery.ModuleSpec(name, _Loader(), is_package=True)
        return None


def install():
    if not REFERENCE_ROOT:
        raise RuntimeError("set AIMET_REFERENCE_ROOT to the checkout of the reference")
    if not os.path.isdir(REFERENCE_ROOT):
        raise RuntimeError(f"reference checkout not found at {REFERENCE_ROOT}")
    if not any(isinstance(f, _Finder) for f in sys.meta_path):
        sys.meta_path.append(_Finder())
        import onnx
        import onnx.defs

        onnx.defs.onnx_opset_version = lambda: 0
        onnx.defs = sys.modules["onnx.defs"]
    for sub in ("TrainingExtensions/torch/src/python", "TrainingExtensions/common/src/python"):
        p = os.path.join(REFERENCE_ROOT, sub)
        if p not in sys.path:
            sys.path.insert(0, p)
