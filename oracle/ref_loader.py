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


def reference_root():
    """Checkout of the reference project: the SSCONV_REFERENCE environment variable, else
    `reference_path` of BASELINE.json at the repository root, else None.  Only the builder of the
    checker and the fixture generator need it; nothing that runs on a GPU box reads the checkout."""
    env = os.environ.get("SSCONV_REFERENCE")
    if env:
        return env
    try:
        import json
        with open(os.path.join(os.path.dirname(_HERE), "BASELINE.json")) as f:
            return json.load(f).get("reference_path")
    except Exception:
        return None


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
