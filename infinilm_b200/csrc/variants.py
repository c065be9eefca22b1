"""Every (source, macro definitions) pair the package can ask for; `build()` compiles them all."""


def all_variants():
    from . import build
    return [(name, None) for name in build.all_sources()]
