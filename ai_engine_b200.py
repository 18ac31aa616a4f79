"""Import alias: the package folder is `ai-engine_b200/`, whose name Python cannot
import as written; `import ai_engine_b200` loads that folder as a package."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ai-engine_b200")
_spec = importlib.util.spec_from_file_location(
    "ai_engine_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["ai_engine_b200"] = _mod
_spec.loader.exec_module(_mod)
