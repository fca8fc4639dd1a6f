"""Loads the `llama.rust_b200` package (its directory name has a dot) for the tests."""
import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load():
    if "llama_rust_b200" in sys.modules:
        return sys.modules["llama_rust_b200"]
    path = os.path.join(ROOT, "llama.rust_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location("llama_rust_b200", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["llama_rust_b200"] = mod
    spec.loader.exec_module(mod)
    return mod
