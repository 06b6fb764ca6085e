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


class TinyBlock(torch.nn.Module):
    def __init__(self, d):
        super().__init__()
        self.up = torch.nn.Linear(d, 2 * d)
        self.down = torch.nn.Linear(2 * d, d)

    def forward(self, h):
        return h + self.down(torch.nn.functional.gelu(self.up(h)))


class TinyLM(torch.nn.Module):
    """A small live language model (embedding, residual MLP blocks, tied-free head)
    for the end-to-end objectives: `forward(input_ids, labels=None)` returns an
    object with `.logits` and, given labels, the next-token cross-entropy `.loss`,
    like a HuggingFace causal LM."""

    def __init__(self, vocab=48, d=32, n_layers=2, ctx=16, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.embed = torch.nn.Embedding(vocab, d)
        self.layers = torch.nn.ModuleList([TinyBlock(d) for _ in range(n_layers)])
        self.head = torch.nn.Linear(d, vocab, bias=False)
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * (0.5 if p.ndim == 1 else p.shape[-1] ** -0.5))
        self.config = types.SimpleNamespace(num_hidden_layers=n_layers)
        self.dummy_inputs = {"input_ids": torch.zeros(1, ctx, dtype=torch.long)}

    @property
    def base_model(self):
        return self

    @property
    def device(self):
        return self.embed.weight.device

    def forward(self, input_ids=None, labels=None, **kw):
        h = self.embed(input_ids)
        for layer in self.layers:
            h = layer(h)
        logits = self.head(h)
        loss = None
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(
                logits[:, :-1].reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1))
        return types.SimpleNamespace(logits=logits, loss=loss)


def token_dataset(steps, batch, ctx, vocab=48, seed=3):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (steps * batch, ctx), generator=g)
    return [{"input_ids": row} for row in ids]
