"""Functional minimal HookPoint / HookedRootModule with the interface the reference models use."""
import torch.nn as nn


class HookPoint(nn.Module):
    def __init__(self):
        super().__init__()
        self.fwd_hooks = []
        self.bwd_hooks = []
        self.ctx = {}
        self.name = None

    def add_hook(self, hook, dir="fwd", is_permanent=False, level=None, prepend=False):
        def full_hook(module, module_input, module_output):
            return hook(module_output, hook=self)

        if dir == "fwd":
            handle = self.register_forward_hook(full_hook, prepend=prepend)
            self.fwd_hooks.append((handle, is_permanent))
        else:
            raise NotImplementedError("backward hooks are not provided by this stand-in")

    def remove_hooks(self, dir="fwd", including_permanent=False, level=None):
        keep = []
        for handle, perm in self.fwd_hooks:
            if perm and not including_permanent:
                keep.append((handle, perm))
            else:
                handle.remove()
        self.fwd_hooks = keep

    def clear_context(self):
        self.ctx = {}

    def forward(self, x):
        return x

    def layer(self):
        return int(self.name.split(".")[1])


class HookedRootModule(nn.Module):
    def __init__(self, *args):
        super().__init__()
        self.is_caching = False
        self.context_level = 0

    def setup(self):
        self.mod_dict = {}
        self.hook_dict = {}
        for name, module in self.named_modules():
            if name == "":
                continue
            module.name = name
            self.mod_dict[name] = module
            if isinstance(module, HookPoint):
                self.hook_dict[name] = module

    def hook_points(self):
        return self.hook_dict.values()

    def reset_hooks(self, clear_contexts=True, direction="both", including_permanent=False, level=None):
        for hp in self.hook_points():
            hp.remove_hooks("fwd", including_permanent=including_permanent)
            if clear_contexts:
                hp.clear_context()
