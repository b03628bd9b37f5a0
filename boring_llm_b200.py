"""Import shim: `import boring_llm_b200` loads the package kept in the folder `boring-llm_b200/`.

A folder name with a hyphen cannot be written in an import statement, so this module
replaces itself in `sys.modules` with the real package, loaded from that folder, and
submodules (`boring_llm_b200.config`, ...) resolve inside it.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "boring-llm_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
