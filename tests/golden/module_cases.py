"""The module / checkpoint scenario shared by make_golden_modules.py (run on the unmodified
reference) and tests/test_gpu_modules.py (run on litenn_b200): a nested Module with python
variables, lists and dicts of sub-modules and an SGD optimizer with momentum as a saveable,
following the procedure of the reference's own Module_test (litenn/core/test/test.py:42-145)
with seeded tensor contents instead of constants.  Written against the `nn` namespace only.
"""
import numpy as np


def build(nn):
    class Block(nn.Module):
        def __init__(self, include_self=True):
            if include_self:
                self.mod = Block(include_self=False)
            self.a = 1
            self.l = [1, 1]
            self.tag = "first"
            self.scale = 0.5
            self.conv1 = nn.Conv2D(2, 3, 3)
            self.list_of_convs = [nn.Conv2D(3, 3, 1), nn.Conv2D(3, 2, 3, use_bias=False)]
            self.dict_of_layers = {0: nn.Conv2D(2, 2, 1), "asd": nn.Dense(4, 5)}
            self._hidden = 7        # names starting with _ are not saved

        def forward(self, x):
            x = self.conv1(x)
            x = self.list_of_convs[0](x)
            return self.list_of_convs[1](x)

    class Trainer(nn.Module):
        def __init__(self):
            self.mod1 = Block()
            self.opt1 = nn.optimizer.SGD(self.mod1.trainables(), momentum=0.9, lr=0.01)

    return Trainer()


def fill(trainer, seed=11):
    """Seeded contents for every trainable tensor, in trainables() order."""
    rng = np.random.default_rng(seed)
    for t in trainer.mod1.trainables():
        t.set(rng.standard_normal(tuple(t.shape)).astype(np.float32))


def train_input(seed=12):
    return np.random.default_rng(seed).standard_normal((2, 2, 6, 6)).astype(np.float32)


def train_step(nn, trainer, x_np):
    """loss = mean(mod1(x)); one SGD step."""
    opt = trainer.opt1
    opt.zero_grad()
    y = trainer.mod1(nn.Tensor_from_value(x_np))
    loss = y.mean()
    loss.backward()
    opt.step()
    return loss.np()


# ---- optimizer update rules ------------------------------------------------------------------
OPTIMIZERS = {
    "sgd_plain": ("SGD", dict(lr=0.05)),
    "sgd_momentum": ("SGD", dict(momentum=0.9, lr=0.05)),
    "sgd_nesterov_decay": ("SGD", dict(momentum=0.8, nesterov=True, lr=0.05, lr_decay=0.3)),
    "sgd_dropout": ("SGD", dict(momentum=0.5, lr=0.05, lr_dropout=0.6)),
    "rmsprop": ("RMSprop", dict(rho=0.9, lr=0.01)),
    "rmsprop_decay_dropout": ("RMSprop", dict(rho=0.95, lr=0.01, lr_decay=0.1, lr_dropout=0.3)),
    "adam": ("Adam", dict(beta_1=0.9, beta_2=0.999, lr=0.01)),
    "adam_dropout": ("Adam", dict(beta_1=0.8, beta_2=0.99, lr=0.02, lr_dropout=0.5)),
    "sgd_clipnorm": ("SGD", dict(lr=0.05, clipnorm=1.5)),
}


def run_optimizer(nn, name, steps=3):
    """Three steps of one optimizer on two seeded tensors with seeded gradients; the host random
    stream is seeded so that the learning-rate-dropout seeds are the same on both sides."""
    cls, kw = OPTIMIZERS[name]
    rng = np.random.default_rng(sum(map(ord, name)))
    ts = [nn.Tensor_from_value(rng.standard_normal(shape).astype(np.float32)) for shape in ((37,), (4, 9))]
    opt = getattr(nn.optimizer, cls)(ts, **kw)
    np.random.seed(1234)
    for _ in range(steps):
        for t in ts:
            t.get_grad().set(rng.standard_normal(tuple(t.shape)).astype(np.float32))
        opt.step()
    out = {f"t{i}": t.np() for i, t in enumerate(ts)}
    for k, v in opt.dump_state().items():
        if isinstance(v, tuple) and v[0] == "np.ndarray":
            out[f"state/{len(out)}"] = v[1]
    out["iteration"] = np.asarray(opt.iteration)
    return out
