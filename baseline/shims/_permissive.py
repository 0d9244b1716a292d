"""Stand-ins for third-party packages that the reference imports at module import time but
that are absent from this offline image (hydra, omegaconf, accelerate, peft, deepspeed,
decord, librosa, soundfile, jsonlines, qwen_vl_utils, av).  None of them sits on the timed
training path of the reference's fsdp2 trainer; the few functions that ARE called
(``accelerate.utils.send_to_device``, ``init_empty_weights``) are implemented for real.
Any other attribute resolves to an inert placeholder so that ``from pkg import Name`` works.
The reference's own source is used unmodified."""
import sys
import types


class _Placeholder:
    def __init__(self, *a, **k):
        pass

    def __call__(self, *a, **k):
        if len(a) == 1 and callable(a[0]) and not k:
            return a[0]  # used as a decorator
        return _Placeholder()

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return _Placeholder()

    def __iter__(self):
        return iter(())

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False

    def __mro_entries__(self, bases):
        return (object,)


class PermissiveModule(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        full = self.__name__ + "." + name
        if full in sys.modules:
            return sys.modules[full]
        cls = type(name, (_Placeholder,), {})
        setattr(self, name, cls)
        return cls


class _SubmoduleFinder:
    """Makes ``import pkg.any.sub.module`` succeed for every stand-in package, so that a
    third-party library which probes one of them (Liger imports ``peft.utils.other`` when it
    sees a ``peft`` module) does not fail on a submodule nobody listed."""

    roots: set = set()

    @classmethod
    def find_spec(cls, fullname, path=None, target=None):
        from importlib.machinery import ModuleSpec

        if fullname.split(".", 1)[0] not in cls.roots or fullname in sys.modules:
            return None
        return ModuleSpec(fullname, cls, is_package=True)

    @staticmethod
    def create_module(spec):
        m = PermissiveModule(spec.name)
        m.__path__ = []
        return m

    @staticmethod
    def exec_module(module):
        pass


def install(name, submodules=(), attrs=None):
    from importlib.machinery import ModuleSpec

    _SubmoduleFinder.roots.add(name)
    if _SubmoduleFinder not in sys.meta_path:
        sys.meta_path.append(_SubmoduleFinder)

    mod = PermissiveModule(name)
    mod.__path__ = []  # behaves as a package
    mod.__version__ = "0.0.0"
    mod.__spec__ = ModuleSpec(name, None, is_package=True)
    sys.modules[name] = mod
    for sub in submodules:
        m = PermissiveModule(name + "." + sub)
        m.__path__ = []
        m.__spec__ = ModuleSpec(name + "." + sub, None, is_package=True)
        sys.modules[name + "." + sub] = m
        parent = sys.modules[(name + "." + sub).rsplit(".", 1)[0]]
        setattr(parent, sub.rsplit(".", 1)[-1], m)
    for k, v in (attrs or {}).items():
        target, _, attr = k.rpartition(".")
        setattr(sys.modules[name + ("." + target if target else "")], attr, v)
    return mod
