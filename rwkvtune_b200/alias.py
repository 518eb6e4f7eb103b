"""Run code written against the reference's import name (``rwkvtune``) on this package.

Every script and notebook of the reference starts with ``from rwkvtune import ...``
(``rwkvtune/__init__.py:24-93``, ``examples/train_sft_single_gpu.py``).  This module makes
those imports resolve to :mod:`rwkvtune_b200` without copying or renaming anything:

    python -m rwkvtune_b200.alias path/to/script.py [script args...]    # run a script unmodified
    python -m rwkvtune_b200.alias -m some.module [args...]               # run a module unmodified

or, inside a program::

    import rwkvtune_b200.alias as alias; alias.install()
    from rwkvtune import AutoModel, SFTTrainer            # rwkvtune_b200.AutoModel, ...
    from rwkvtune.peft import LoraConfig                  # rwkvtune_b200.peft.LoraConfig

``install()`` puts a finder at the front of ``sys.meta_path`` that maps ``rwkvtune`` and every
``rwkvtune.x.y`` to ``rwkvtune_b200`` / ``rwkvtune_b200.x.y`` (the same module object under both
names).  It refuses to install when a real ``rwkvtune`` distribution is importable (for example the
unmodified reference that the benchmark's comparison arm installs into its own directory): the two
must never be mixed in one process.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import importlib.util
import runpy
import sys

ALIAS, TARGET = "rwkvtune", "rwkvtune_b200"


class AliasConflict(ImportError):
    pass


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target_name: str):
        self.target_name = target_name

    def create_module(self, spec):
        return importlib.import_module(self.target_name)   # the real module object, shared under both names

    def exec_module(self, module):   # already executed under its own name
        return None


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if fullname != ALIAS and not fullname.startswith(ALIAS + "."):
            return None
        target_name = TARGET + fullname[len(ALIAS):]
        try:
            real = importlib.util.find_spec(target_name)
        except (ImportError, ValueError):
            real = None
        if real is None:
            return None
        spec = importlib.machinery.ModuleSpec(fullname, _AliasLoader(target_name),
                                              is_package=real.submodule_search_locations is not None)
        return spec


def _real_distribution_present() -> bool:
    for finder in sys.meta_path:
        if isinstance(finder, _AliasFinder):
            continue
        try:
            spec = finder.find_spec(ALIAS, None) if hasattr(finder, "find_spec") else None
        except Exception:
            spec = None
        if spec is not None:
            return True
    return False


def installed() -> bool:
    return any(isinstance(f, _AliasFinder) for f in sys.meta_path)


def install() -> None:
    """Make ``import rwkvtune[.sub.module]`` resolve to this package.  Idempotent."""
    if installed():
        return
    loaded = sys.modules.get(ALIAS)
    if loaded is not None and getattr(loaded, "__name__", "") != TARGET:
        raise AliasConflict("a different 'rwkvtune' package is already imported in this process")
    if _real_distribution_present():
        raise AliasConflict("a real 'rwkvtune' package is importable from sys.path; refusing to shadow it "
                            "(remove its directory from sys.path / PYTHONPATH to use the alias)")
    sys.meta_path.insert(0, _AliasFinder())


def uninstall() -> None:
    sys.meta_path[:] = [f for f in sys.meta_path if not isinstance(f, _AliasFinder)]
    for name in [n for n in sys.modules if n == ALIAS or n.startswith(ALIAS + ".")]:
        del sys.modules[name]


def main(argv=None) -> None:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit(__doc__)
    install()
    if argv[0] == "-m":
        if len(argv) < 2:
            raise SystemExit("usage: python -m rwkvtune_b200.alias -m module [args...]")
        sys.argv = argv[1:]
        runpy.run_module(argv[1], run_name="__main__", alter_sys=True)
    else:
        sys.argv = argv
        runpy.run_path(argv[0], run_name="__main__")


if __name__ == "__main__":
    main()
