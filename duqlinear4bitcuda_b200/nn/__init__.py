from .linear import Linear4bitSQ, Linear4bitASQ, Linear4bitDUSQ, LinearQuant4bitDUASQ, LinearQuant8bitASQ  # noqa: F401
from .quantizer import SymQuantizer, AsymQuantizer, AsymQuantizer8bit  # noqa: F401
from .matmul import AsymQuantMatMul, SymQuantMatMul  # noqa: F401
