"""A small host-side mirror of popcorn's op registry, for processes without popcorn.

popcorn's call surface for an op is (src/popcorn/core/dispatcher.py:204-345):

    op(*args, backend="name")        force one backend for the call
    op["name"](*args)                the same through the implementation object
    with op["name"]: op(*args)       scope every call in the block
    op.register("name", source="pkg.mod.fn", predicate=..., forward_only=...)
    op.available_backends()

and ops live in a module-level ``KERNELS`` dict filled by ``register_kernel``
(:465-481).  This module reproduces exactly that surface, and nothing of
popcorn's tuner, evidence store or torch reference: here an op is only its
signature plus the backends registered on it, and a call with no eligible
backend is an error rather than a fall-back to PyTorch arithmetic.  When popcorn
itself is importable, use ``popcorn_b200.plugin.register()`` to attach the same
callables to popcorn's own registry instead.
"""

from __future__ import annotations

import importlib
import inspect
import re
from collections.abc import Callable
from contextvars import ContextVar
from types import ModuleType
from typing import Any

import torch

KERNELS: dict[str, "Op"] = {}

_NAME = re.compile(r"^[a-z0-9][a-z0-9_-]*(:[a-z0-9][a-z0-9_-]*)?$")  # dispatcher.py:30


class DispatchError(RuntimeError):
    """No backend can serve the call, or the named one does not exist / declined it."""


def resolve(path: str) -> Any:
    """Import a dotted path, attributes winning over submodules (src/popcorn/core/sources.py:106-125)."""
    head, *rest = path.split(".")
    found: Any = importlib.import_module(head)
    prefix = head
    for part in rest:
        prefix = f"{prefix}.{part}"
        try:
            found = getattr(found, part)
        except AttributeError:
            if not isinstance(found, ModuleType):
                raise
            found = importlib.import_module(prefix)
    return found


class Implementation:
    """One backend of an op: a lazily imported `source`, an optional adapter in front of it."""

    def __init__(self, op: "Op", name: str, source: str | None, predicate: Callable[..., bool] | None, forward_only: bool) -> None:
        if not _NAME.match(name):
            raise ValueError(f"invalid backend name {name!r}")
        self.op, self.name, self.source = op, name, source
        self.predicate, self.forward_only = predicate, forward_only
        self.adapter: Callable[..., Any] | None = None
        self._fn: Callable[..., Any] | None = None

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        return self.op(*args, backend=self.name, **kwargs)

    def __enter__(self) -> "Op":
        self.op._scope.set((*self.op._scope.get(), self.name))
        return self.op

    def __exit__(self, *exc: object) -> None:
        self.op._scope.set(self.op._scope.get()[:-1])

    def __repr__(self) -> str:
        return f"<{self.op.name}:{self.name}{' fwd-only' if self.forward_only else ''}>"

    def rejects(self, arguments: dict[str, Any]) -> str | None:
        """Why this backend must decline the call, or None (dispatcher.py:126-137)."""
        if self.forward_only and torch.is_grad_enabled() and any(
            isinstance(v, torch.Tensor) and v.requires_grad for v in arguments.values()
        ):
            return "no backward implementation"
        if self.predicate is not None and not self.predicate(**arguments):
            return f"rejected by {getattr(self.predicate, '__name__', 'predicate')}"
        return None

    def invoke(self, arguments: dict[str, Any]) -> Any:
        if self._fn is None and self.source is not None:
            self._fn = resolve(self.source)
        args = tuple(arguments[name] for name in self.op.params)
        if self.adapter is not None:
            return self.adapter(*args)
        if self._fn is None:
            raise DispatchError(f"{self.op.name}:{self.name}: registration has neither adapter nor source")
        return self._fn(*args)


class Op:
    """An op declared by its signature; callable like popcorn's Dispatcher."""

    def __init__(self, declaration: Callable[..., Any], name: str | None = None) -> None:
        self.name = name or declaration.__name__
        self.__name__ = self.name
        self.__doc__ = declaration.__doc__
        self.signature = inspect.signature(declaration)
        self.params = tuple(self.signature.parameters)
        self._impls: list[Implementation] = []
        self._scope: ContextVar[tuple[str, ...]] = ContextVar(f"popcorn_b200.{self.name}", default=())

    def register(
        self, name: str, source: str | None = None, predicate: Callable[..., bool] | None = None, forward_only: bool = False
    ) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
        if any(impl.name == name for impl in self._impls):
            raise ValueError(f"{self.name}: backend {name!r} already registered")
        impl = Implementation(self, name, source, predicate, forward_only)
        self._impls.append(impl)

        def attach(adapter: Callable[..., Any]) -> Callable[..., Any]:
            names = tuple(inspect.signature(adapter).parameters)
            if names != self.params:
                self._impls.remove(impl)
                raise TypeError(f"{self.name}:{name}: parameters must be exactly {list(self.params)}, got {list(names)}")
            impl.adapter = adapter
            return adapter

        return attach

    def available_backends(self) -> tuple[str, ...]:
        return tuple(impl.name for impl in self._impls)

    def __getitem__(self, name: str) -> Implementation:
        for impl in self._impls:
            if impl.name == name:
                return impl
        raise DispatchError(f"{self.name}: unknown backend {name!r}; available: {', '.join(self.available_backends())}")

    def __call__(self, *args: Any, backend: str | None = None, **kwargs: Any) -> Any:
        bound = self.signature.bind(*args, **kwargs)
        bound.apply_defaults()
        arguments = dict(bound.arguments)
        scoped = self._scope.get()
        forced = backend or (scoped[-1] if scoped else None)
        if forced is not None:
            impl = self[forced]
            if reason := impl.rejects(arguments):
                raise DispatchError(f"{self.name}: backend {forced!r} rejected call: {reason}")
            return impl.invoke(arguments)
        for impl in self._impls:  # registration order
            if impl.rejects(arguments) is None:
                return impl.invoke(arguments)
        raise DispatchError(f"{self.name}: no registered backend accepts this call")

    def __repr__(self) -> str:
        return f"{self.name}{self.signature}\n" + "\n".join(f"  {impl.name}" for impl in self._impls)


def register_kernel(declaration: Callable[..., Any] | None = None, *, name: str | None = None) -> Any:
    """Declare an op from a function's signature and docstring (its body is never run)."""

    def wrap(fn: Callable[..., Any]) -> Op:
        op = Op(fn, name)
        if op.name in KERNELS:
            raise ValueError(f"kernel {op.name!r} already registered")
        KERNELS[op.name] = op
        return op

    return wrap(declaration) if declaration is not None else wrap
