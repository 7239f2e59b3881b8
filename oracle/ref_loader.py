"""Load the reference's own compiled extension (oracle/_ref/_ext*.so, built by
oracle/build_ref.py from SS_Conv_lib/src).  Test infrastructure only.

load_ref_ext() returns the module exporting the reference's 32 functions
(SS_Conv_lib/src/ss_conv_ops_api.cpp:15-55) or None when it has not been built.
"""
import importlib.util
import os
import sysconfig

_HERE = os.path.dirname(os.path.abspath(__file__))
_CACHE = {}


def ref_ext_path():
    return os.path.join(_HERE, "_ref", "_ext" + sysconfig.get_config_var("EXT_SUFFIX"))


def load_ref_ext():
    if "m" in _CACHE:
        return _CACHE["m"]
    path = ref_ext_path()
    mod = None
    if os.path.exists(path):
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        spec = importlib.util.spec_from_file_location("_ext", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    _CACHE["m"] = mod
    return mod
