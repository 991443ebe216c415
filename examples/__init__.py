"""User-level kernel definitions (arrangement + application) used by the tests and the benchmark."""

import importlib.util
import pathlib

_DEFINITIONS = pathlib.Path(__file__).resolve().parent / "definitions.py"


def load_definitions(front_end: str = "ninetoothed_b200"):
    """Execute ``definitions.py`` against the front-end package named ``front_end``.

    ``"ninetoothed_b200"`` gives this library's kernels; ``"ninetoothed"`` (the reference
    package, when it is importable) gives the same definitions compiled by the reference.
    The module is loaded from its file, so ``inspect.getsource`` works on its functions.
    """
    spec = importlib.util.spec_from_file_location(f"examples._definitions_for_{front_end}", _DEFINITIONS)
    module = importlib.util.module_from_spec(spec)
    module.__front_end__ = front_end
    spec.loader.exec_module(module)
    return module
