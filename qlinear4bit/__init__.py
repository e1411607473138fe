"""Drop-in alias: `import qlinear4bit.nn`, `qlinear4bit.tools.tensor_utils`, `qlinear4bit._CUDA`
resolve to the duqlinear4bitcuda_b200 implementation, so code written against the reference
package imports unchanged."""
import importlib
import sys

import duqlinear4bitcuda_b200 as _impl

for _name in ("_CUDA", "tools", "tools.quantization", "tools.tensor_utils", "nn", "nn.quantizer", "nn.linear", "nn.matmul"):
    _mod = importlib.import_module("duqlinear4bitcuda_b200." + _name)
    sys.modules["qlinear4bit." + _name] = _mod
    if "." not in _name:
        globals()[_name] = _mod

__version__ = _impl.__version__
