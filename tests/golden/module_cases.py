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
