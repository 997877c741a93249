"""Name -> class/function registries.

Every pluggable thing in the engine (architectures, embeddings, output layers, mixers,
feed-forwards, norms, position encodings, block arrangements, activations) lives in one of
these registries under a string name.  A model description refers to parts by
name only, so a new part is added by registering it; no framework file has to
change.

Same role as simply/utils/registry.py:25-102 (RootRegistry: register / get /
keys / unregister, duplicate names are an error), but one small instance per
kind of thing instead of one class-level dict with namespaces.
"""

from __future__ import annotations

from typing import Any, Callable, Generic, Iterator, TypeVar

T = TypeVar("T")


class Registry(Generic[T]):
  """A dictionary from names to registered objects with loud failures."""

  def __init__(self, kind: str):
    self.kind = kind
    self._items: dict[str, T] = {}

  def register(self, name: str, item: T | None = None, *, replace: bool = False) -> Any:
    """Registers `item` under `name`; usable as a decorator when item is None."""

    def _do(obj: T) -> T:
      if not name:
        raise ValueError(f"{self.kind}: a registered name must not be empty")
      if name in self._items and not replace:
        raise ValueError(f"{self.kind}: duplicate name {name!r}")
      self._items[name] = obj
      return obj

    if item is None:
      return _do
    return _do(item)

  def unregister(self, name: str) -> None:
    self._items.pop(name, None)

  def get(self, name: str) -> T:
    try:
      return self._items[name]
    except KeyError:
      known = ", ".join(sorted(self._items)) or "<none>"
      raise KeyError(f"{self.kind}: unknown name {name!r}; registered: {known}") from None

  def __contains__(self, name: str) -> bool:
    return name in self._items

  def __iter__(self) -> Iterator[str]:
    return iter(sorted(self._items))

  def keys(self) -> list[str]:
    return sorted(self._items)


# One registry per kind of part.  Values are classes (parts) or callables.
ARCHITECTURES: Registry[Any] = Registry("architecture")
EMBEDDINGS: Registry[Any] = Registry("embedding")
HEADS: Registry[Any] = Registry("head")
MIXERS: Registry[Any] = Registry("mixer")
FEED_FORWARDS: Registry[Any] = Registry("feed_forward")
NORMS: Registry[Any] = Registry("norm")
POSITION_ENCODINGS: Registry[Any] = Registry("position_encoding")
BLOCKS: Registry[Any] = Registry("block")
ACTIVATIONS: Registry[int] = Registry("activation")
