"""``nn.Module`` with the reference's method names on top of ``torch.nn.Module``.

Reference: infini_train/include/nn/modules/module.h:12-45 and
src/nn/modules/module.cc.  Deliberate differences: tied tensors are listed once
by ``Parameters()`` and stay tied across ``To(device)`` (the reference
duplicates them, module.cc:12-19, and breaks the tie on a device move, :58-71).
"""
from __future__ import annotations

from typing import Callable, Dict, List

import torch


class Module(torch.nn.Module):
    kUndefinedType = "Undefined"

    def type(self) -> str:  # noqa: A003  (reference name)
        return getattr(self, "kType", self.__class__.__name__)

    # ---- parameters -------------------------------------------------------------
    def Parameters(self) -> List[torch.Tensor]:
        return list(self.parameters())

    def has_parameter(self, name: str) -> bool:
        return name in self._parameters and self._parameters[name] is not None

    def parameter(self, name: str) -> torch.Tensor:
        if not self.has_parameter(name):
            raise KeyError(f"no parameter named {name!r} in {self.type()}")
        return self._parameters[name]

    def mutable_parameter(self, name: str) -> torch.Tensor:
        return self.parameter(name)

    # ---- sub-modules ---------------------------------------------------------------
    def modules_list(self) -> List["Module"]:
        """All sub-modules, depth first (the reference's ``modules()``)."""
        return [m for _, m in self.named_modules() if m is not self]

    def module(self, name: str) -> "Module":
        return self.get_submodule(name)

    def mutable_module(self, name: str) -> "Module":
        return self.get_submodule(name)

    # ---- state ----------------------------------------------------------------------
    def StateDict(self) -> Dict[str, torch.Tensor]:
        """Dotted-name -> tensor map; tied tensors appear under every name that reaches them."""
        return dict(self.named_parameters(remove_duplicate=False))

    def To(self, device) -> "Module":
        return self.to(device)

    def Apply(self, fn: Callable[["Module"], None]) -> "Module":
        """Post-order traversal, children before the module itself."""
        return self.apply(fn)

    def Forward(self, inputs):
        """Reference calling convention: a list of tensors in, a list of tensors out."""
        out = self.forward(*inputs)
        return list(out) if isinstance(out, (tuple, list)) else [out]
