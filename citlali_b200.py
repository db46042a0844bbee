"""Import alias: ``import citlali_b200`` loads the package kept in ``citlali-llm-engine_b200/``.

The package folder carries the project's name, which is not a valid Python
identifier; this module replaces itself in ``sys.modules`` with that package.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "citlali-llm-engine_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
