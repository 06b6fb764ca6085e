"""A stand-in for the language model the Trainer hooks into: one ModuleList of
layers whose outputs are stored activation batches (no language model, dataset
or tokenizer is involved in the tests)."""

import types

import torch


class FakeLayer(torch.nn.Module):
    def __init__(self, owner, index):
        super().__init__()
        object.__setattr__(self, "_owner", owner)
        self.index = index

    def forward(self, h):
        return self._owner.activation(self.index)


class FakeModel(torch.nn.Module):
    """acts: [steps, B, T, D] (one hooked layer) or a list of such tensors (one
    per layer). Every forward call advances to the next stored batch; the first
    call (the Trainer's width probe) does not consume one."""

    def __init__(self, acts, device="cpu"):
        super().__init__()
        acts = acts if isinstance(acts, (list, tuple)) else [acts]
        self.acts = [a.to(device) for a in acts]
        self.config = types.SimpleNamespace(num_hidden_layers=len(self.acts))
        self.layers = torch.nn.ModuleList([FakeLayer(self, i) for i in range(len(self.acts))])
        self.cursor = -1
        self._device = torch.device(device)
        T = self.acts[0].shape[2]
        self.dummy_inputs = {"input_ids": torch.zeros(1, T, dtype=torch.long)}

    @property
    def base_model(self):
        return self

    @property
    def device(self):
        return self._device

    def activation(self, layer):
        a = self.acts[layer]
        return a[min(max(self.cursor, 0), a.shape[0] - 1)]

    def forward(self, input_ids=None, **kw):
        h = input_ids
        for layer in self.layers:
            h = layer(h)
        self.cursor += 1
        return h


def dataset(steps, batch, ctx):
    return [{"input_ids": torch.zeros(ctx, dtype=torch.long)} for _ in range(steps * batch)]
