"""Loader for the in-tree sm_100a extension (filled in by the kernel build)."""


def ensure_loaded() -> None:
    raise RuntimeError("the sm_100a extension has not been built: run `python -c 'import __graft_entry__ as g; g.build()'`")
