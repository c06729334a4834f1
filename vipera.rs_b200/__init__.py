"""A small, whole inference engine for one B200 GPU and one architecture family
(the Qwen2 / Qwen2.5 dense decoder), built from parts so that another can be added.

    from vipera_rs_b200 import Engine, SamplingParams
    engine = Engine("path/to/model", dtype="bfloat16")
    result = engine.generate([[151, 2040, 17]], SamplingParams(max_new_tokens=16))[0]
"""
from . import errors
from .config import load_config
from .engine import Engine, Generation, StepReport, load_model, random_model, write_random_model
from .sampling import SamplingParams

__all__ = ["errors", "load_config", "Engine", "Generation", "StepReport", "SamplingParams",
           "load_model", "random_model", "write_random_model"]


def _load_plugins() -> None:
    """Import the files or modules listed in VIPERA_PLUGINS (separated like PATH) and call their
    ``register()``: the way a process that did not define a part itself (a command-line tool)
    learns of parts and architectures registered from outside the package."""
    import importlib
    import importlib.util
    import os
    import sys

    for item in filter(None, os.environ.get("VIPERA_PLUGINS", "").split(os.pathsep)):
        if item.endswith(".py") and os.path.exists(item):
            folder, name = os.path.dirname(os.path.abspath(item)), os.path.splitext(os.path.basename(item))[0]
            if folder not in sys.path:
                sys.path.insert(0, folder)
            module = importlib.import_module(name)
        else:
            module = importlib.import_module(item)
        register = getattr(module, "register", None)
        if callable(register):
            register()


_load_plugins()
