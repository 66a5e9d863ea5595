"""Name -> class registry with aliases, the lookup mechanism behind
``BaseCompressor.register(name=...)`` / ``TransformFactory.register(...)`` (registry/registry.py:68-361).
Each direct subclass of RegistryMixin that is used as a root keeps its own table."""
from typing import Dict, List, Optional, Type, Union

__all__ = ["RegistryMixin", "standardize_lookup_name"]


def standardize_lookup_name(name: str) -> str:
    """Names compare case-insensitively with '-', '_' and ' ' treated alike."""
    return name.replace("_", "-").replace(" ", "-").lower()


_TABLES: Dict[type, Dict[str, type]] = {}
_ALIASES: Dict[type, Dict[str, str]] = {}


class RegistryMixin:
    registry_requires_subclass: bool = False

    @classmethod
    def register(cls, name: Optional[str] = None, alias: Union[List[str], str, None] = None):
        def decorator(value: type):
            cls.register_value(value, name=name, alias=alias)
            return value

        return decorator

    @classmethod
    def register_value(cls, value: type, name: Optional[str] = None, alias: Union[List[str], str, None] = None):
        name = standardize_lookup_name(name if name is not None else value.__name__)
        aliases = [alias] if isinstance(alias, str) else list(alias or [])
        if cls.registry_requires_subclass and not issubclass(value, cls):
            raise ValueError(f"{value} must be a subclass of {cls} to be registered under it")
        table = _TABLES.setdefault(cls, {})
        amap = _ALIASES.setdefault(cls, {})
        if name in table and table[name] is not value:
            raise RuntimeError(f"'{name}' is already registered under {cls.__name__} as {table[name]}")
        table[name] = value
        for a in [name] + [standardize_lookup_name(a) for a in aliases]:
            if a in amap and amap[a] != name:
                raise KeyError(f"alias '{a}' already points at '{amap[a]}'")
            amap[a] = name

    @classmethod
    def get_value_from_registry(cls, name: str) -> type:
        key = standardize_lookup_name(name)
        for root in cls.__mro__:
            amap = _ALIASES.get(root)
            if amap and key in amap:
                return _TABLES[root][amap[key]]
        if ":" in name:  # "module.path:ClassName"
            import importlib

            mod, attr = name.split(":", 1)
            return getattr(importlib.import_module(mod), attr)
        raise KeyError(f"Unable to find '{name}' registered under {cls.__name__}; known: {cls.registered_names()}")

    @classmethod
    def load_from_registry(cls, name: str, **constructor_kwargs):
        return cls.get_value_from_registry(name)(**constructor_kwargs)

    @classmethod
    def registered_names(cls) -> List[str]:
        return sorted(n for root in cls.__mro__ for n in _TABLES.get(root, {}))

    @classmethod
    def registered_aliases(cls) -> List[str]:
        return sorted(n for root in cls.__mro__ for n in _ALIASES.get(root, {}))
