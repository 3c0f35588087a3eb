"""A small model library with generation for one NVIDIA B200: the Llama / SmolLM2 decoder.

    from scriptling_llm_lib_b200 import llm
    ids = llm.generate(model_dir, prompt_ids, 32, "greedy", temperature=0.0)
"""
from . import models  # noqa: F401  (registers the architectures)

VERSION = "0.1.0"
__all__ = ["VERSION", "llm"]


def __getattr__(name):
    if name == "llm":
        import importlib
        return importlib.import_module(".llm", __name__)
    raise AttributeError(name)
