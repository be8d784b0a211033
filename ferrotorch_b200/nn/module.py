"""``Module`` base class, ``Parameter`` / ``Buffer``, containers, hooks and the ``derive_module`` decorator.

``Module`` extends ``torch.nn.Module`` with the reference's method names (``parameters_mut``, ``is_training``,
``to_device``, ``apply_to_parameters``, ``named_children`` ...), so models written against either API work.
``derive_module`` is the counterpart of ``#[derive(Module)]``: fields are declared with ``param()``, ``submodule()`` or
``skip()`` markers and a ``training: bool`` field is mandatory; misuse raises :class:`DeriveError` with the same
diagnostics the proc-macro emits at compile time.

Reference parity: ferrotorch-nn/src/module.rs:10-304, parameter.rs:12, buffer.rs:26, container.rs:36-331,
parameter_container.rs:20-119, hooks.rs:60-104, ferrotorch-nn-derive/src/lib.rs:1-42 and its tests/compile_fail/*.stderr.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Tuple

import torch

from ..errors import FerrotorchError, InvalidArgument

StateDict = Dict[str, torch.Tensor]
Parameter = torch.nn.Parameter


class Reduction(enum.Enum):
    Mean = "mean"
    Sum = "sum"
    None_ = "none"


class Buffer(torch.Tensor):
    """A non-trainable tensor registered on a module (running statistics, masks); saved in the state dict."""

    def __new__(cls, data: torch.Tensor, persistent: bool = True):
        t = torch.Tensor._make_subclass(cls, data.detach(), False)
        t.persistent = persistent
        return t


class Module(torch.nn.Module):
    """Base class of every layer."""

    # -- reference method names --------------------------------------------------------------------
    def parameters_mut(self) -> Iterator[Parameter]:
        return self.parameters()

    def is_training(self) -> bool:
        return self.training

    def to_device(self, device) -> "Module":
        """Move every parameter and buffer (build optimizers afterwards, as with the reference: ferrotorch-nn/src/module.rs:55-63)."""
        return self.to(torch.device(str(device)) if not isinstance(device, torch.device) else device)

    def apply_to_parameters(self, fn: Callable[[Parameter], None]) -> "Module":
        with torch.no_grad():
            for p in self.parameters():
                fn(p)
        return self

    def num_parameters(self, trainable_only: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not trainable_only)

    def __setattr__(self, name: str, value: Any) -> None:
        if isinstance(value, Buffer):
            self.register_buffer(name, value.as_subclass(torch.Tensor), persistent=getattr(value, "persistent", True))
            return
        super().__setattr__(name, value)

    def state_dict_cpu(self) -> StateDict:
        return {k: v.detach().cpu() for k, v in self.state_dict().items()}


class HookHandle:
    def __init__(self, handle):
        self._h = handle

    def remove(self) -> None:
        self._h.remove()


class HookedModule(Module):
    """Wraps a module and exposes forward / forward-pre / backward hooks with removable handles."""

    def __init__(self, inner: torch.nn.Module):
        super().__init__()
        self.inner = inner

    def forward(self, *a, **k):
        return self.inner(*a, **k)

    def register_forward_hook_fn(self, fn) -> HookHandle:
        """``fn(input, output)`` after every forward; a non-None return value replaces the output (hooks.rs:37)."""
        return HookHandle(self.inner.register_forward_hook(lambda _m, inp, out: fn(inp[0] if len(inp) == 1 else inp, out)))

    def register_forward_pre_hook_fn(self, fn) -> HookHandle:
        """``fn(input) -> replacement input or None`` before every forward (hooks.rs:42)."""
        def pre(_m, inp):
            r = fn(inp[0] if len(inp) == 1 else inp)
            return None if r is None else (r if isinstance(r, tuple) else (r,))
        return HookHandle(self.inner.register_forward_pre_hook(pre))

    def register_backward_hook_fn(self, fn) -> HookHandle:
        """``fn(grad_input, grad_output)`` when the gradients of the wrapped module have been computed (hooks.rs:48)."""
        return HookHandle(self.inner.register_full_backward_hook(
            lambda _m, gi, go: fn(gi[0] if len(gi) == 1 else gi, go[0] if len(go) == 1 else go)))


class Sequential(torch.nn.Sequential, Module):
    pass


class ModuleList(torch.nn.ModuleList, Module):
    pass


class ModuleDict(torch.nn.ModuleDict, Module):
    pass


class ParameterList(torch.nn.ParameterList, Module):
    pass


class ParameterDict(torch.nn.ParameterDict, Module):
    pass


# ----------------------------------------------------------------------------------------------------------------------
# derive_module
# ----------------------------------------------------------------------------------------------------------------------
class DeriveError(FerrotorchError, TypeError):
    """Raised at class-definition time for the misuse cases the proc-macro rejects at compile time."""


class _Marker:
    def __init__(self, kinds: Tuple[str, ...], default=dataclasses.MISSING, default_factory=dataclasses.MISSING):
        self.kinds, self.default, self.default_factory = kinds, default, default_factory

    def __or__(self, other: "_Marker") -> "_Marker":
        return _Marker(self.kinds + other.kinds, self.default, self.default_factory)


def param(**kw) -> _Marker:
    """Marks a trainable tensor field (``#[param]``)."""
    return _Marker(("param",), **kw)


def submodule(**kw) -> _Marker:
    """Marks a child module field (``#[submodule]``)."""
    return _Marker(("submodule",), **kw)


def skip(**kw) -> _Marker:
    """Marks a field that the derive ignores (``#[skip]``)."""
    return _Marker(("skip",), **kw)


def derive_module(cls=None, *, dtype_param: Optional[str] = "T"):
    """Class decorator generating ``__init__``, ``parameters``, ``named_parameters``, ``train/eval`` plumbing.

    ::

        @derive_module
        class Affine(Module):
            weight: torch.Tensor = param()
            inner: Module = submodule()
            note: str = skip(default="")
            training: bool = True
            T = float            # the element type parameter (``T: Float`` in the reference)
    """

    def wrap(c):
        if isinstance(c, type) and issubclass(c, enum.Enum):
            raise DeriveError("#[derive(Module)] only supports structs")
        if not isinstance(c, type):
            raise DeriveError("#[derive(Module)] only supports structs")
        if issubclass(c, tuple):
            raise DeriveError("#[derive(Module)] only supports structs with named fields")
        ann = dict(getattr(c, "__annotations__", {}))
        if not ann:
            raise DeriveError("#[derive(Module)] only supports structs with named fields")
        if "training" not in ann or ann["training"] not in (bool, "bool"):
            raise DeriveError("#[derive(Module)] requires a `training: bool` field")
        if dtype_param is not None and not hasattr(c, dtype_param):
            raise DeriveError("#[derive(Module)] requires at least one type parameter (e.g., `T: Float`)")
        fields: List[Tuple[str, str, _Marker]] = []
        for name in ann:
            if name == "training":
                continue
            mk = c.__dict__.get(name)
            if isinstance(mk, _Marker):
                if len(mk.kinds) > 1:
                    raise DeriveError("field cannot have more than one of #[param], #[submodule], #[skip]")
                fields.append((name, mk.kinds[0], mk))
            else:
                fields.append((name, "skip", _Marker(("skip",), default=mk if name in c.__dict__ else dataclasses.MISSING)))
        base = c if issubclass(c, torch.nn.Module) else None
        if base is None:
            raise DeriveError("#[derive(Module)] only supports structs")  # must extend Module

        def __init__(self, *args, **kwargs):
            torch.nn.Module.__init__(self)
            names = [f[0] for f in fields]
            if len(args) > len(names):
                raise TypeError(f"{c.__name__}() takes at most {len(names)} positional arguments")
            vals = dict(zip(names, args))
            for k, v in kwargs.items():
                if k == "training":
                    continue
                if k not in names or k in vals:
                    raise TypeError(f"{c.__name__}() got an unexpected or duplicate argument {k!r}")
                vals[k] = v
            for name, kind, mk in fields:
                if name not in vals:
                    if mk.default is not dataclasses.MISSING:
                        vals[name] = mk.default
                    elif mk.default_factory is not dataclasses.MISSING:
                        vals[name] = mk.default_factory()
                    else:
                        raise TypeError(f"{c.__name__}() missing required field {name!r}")
                v = vals[name]
                if kind == "param":
                    if not isinstance(v, torch.nn.Parameter):
                        v = torch.nn.Parameter(v)
                    self.register_parameter(name, v)
                elif kind == "submodule":
                    if not isinstance(v, torch.nn.Module):
                        raise DeriveError(f"field `{name}` is marked #[submodule] but is not a Module")
                    self.add_module(name, v)
                else:
                    object.__setattr__(self, name, v)
            self.train(kwargs.get("training", True))
            post = getattr(self, "__post_init__", None)
            if post:
                post()

        for name, _, _ in fields:
            if name in c.__dict__ and isinstance(c.__dict__[name], _Marker):
                delattr(c, name)
        c.__init__ = __init__
        c.__derive_fields__ = [(n, k) for n, k, _ in fields]
        return c

    return wrap(cls) if cls is not None else wrap
