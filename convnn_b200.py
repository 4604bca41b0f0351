"""Import alias: ``import convnn_b200`` loads the package that lives in the directory
``convolutional-nearest-neighbor-attention_b200`` (not a valid identifier) and registers
it, with its sub-modules, under the short name."""
import importlib
import os
import sys

_ROOT = os.path.dirname(os.path.abspath(__file__))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)
_LONG = "convolutional-nearest-neighbor-attention_b200"
_pkg = importlib.import_module(_LONG)
for _name, _mod in list(sys.modules.items()):
    if _name == _LONG or _name.startswith(_LONG + "."):
        sys.modules["convnn_b200" + _name[len(_LONG):]] = _mod
sys.modules[__name__] = _pkg
