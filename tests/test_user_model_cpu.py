"""A user's own model, written with stock ``torch.nn`` modules and the reference's
import names (through the opt-in alias): blocks made of ``nn.Linear`` / ``nn.LayerNorm``
children, buffers, empty per-layer constants, a loss callback that returns a tuple.  The
engine must reproduce plain AdamW on it."""
import subprocess
import sys
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import sys
sys.path.insert(0, %r)
import torch, torch.nn as nn
import flextrain_b200.compat
import flextrain
from flextrain.config import init_flextrain_config
from flextrain.ops.adam import FlexTrainAdam

class Block(nn.Module):
    def __init__(self, width):
        super().__init__()
        self.norm = nn.LayerNorm(width)
        self.fc1 = nn.Linear(width, 2 * width)
        self.fc2 = nn.Linear(2 * width, width, bias=False)
        self.register_buffer("gain", torch.tensor(0.5))
    def forward(self, x):
        return x + self.gain * self.fc2(torch.nn.functional.gelu(self.fc1(self.norm(x))))

class Net(nn.Module):
    def __init__(self, width, depth):
        super().__init__()
        self.inp = nn.Linear(8, width)
        self.blocks = nn.ModuleList([Block(width) for _ in range(depth)])
        self.out = nn.Linear(width, 1)

def make(width=32, depth=5):
    torch.manual_seed(0)
    return Net(width, depth)

gen = torch.Generator().manual_seed(1)
data = [(torch.randn(4, 8, generator=gen), torch.randn(4, 1, generator=gen)) for _ in range(6)]

# ---- plain PyTorch
plain = make()
opt = torch.optim.AdamW(plain.parameters(), lr=1e-2, weight_decay=0.0)
want = []
for x, y in data:
    opt.zero_grad()
    total = 0.0
    for i in range(2):                                  # two micro-batches of two samples
        h = plain.inp(x[2 * i:2 * i + 2])
        for b in plain.blocks:
            h = b(h)
        loss = ((plain.out(h) - y[2 * i:2 * i + 2]) ** 2).mean() / 2
        loss.backward()
        total += float(loss.detach())
    opt.step()
    want.append(total)

# ---- the same model through the engine, reference-style script
flextrain.init_distributed(dist_backend="gloo", force_init=False)
init_flextrain_config({"batch_size": 4, "micro_batch_size": 2, "checkpoint_interval": 2,
                       "mixed_precision": {"device_dtype": "fp32"},
                       "split_ratio": {"parameter": [0.5, 0.5], "optimizer": [0.0, 1.0],
                                       "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0], "alpha": 0.25}})
with flextrain.Init(layer_class=Block, num_layers=5):
    model = make()
optimizer = FlexTrainAdam([{"params": list(model.parameters()), "lr": 1e-2, "weight_decay": 0.0}])
cursor = {"step": 0, "mb": 0}
def get_batch():
    x, y = data[cursor["step"]]
    i = cursor["mb"]
    cursor["mb"] += 1
    if cursor["mb"] == 2:
        cursor["mb"], cursor["step"] = 0, cursor["step"] + 1
    return (x[2 * i:2 * i + 2],), (), (y[2 * i:2 * i + 2],)
def pre_process(pre_inputs):
    return (model.inp(pre_inputs[0]),), ()              # no per-layer constants at all
def layer_forward(start, end):
    def run(h):
        for i in range(start, min(end, len(model.blocks))):
            h = model.blocks[i](h)
        return (h,)
    return run
def post_process(passed_down, post_inputs):
    return (model.out(passed_down[0]),)
def loss_fn(outputs, loss_inputs):
    err = ((outputs[0] - loss_inputs[0]) ** 2).mean()
    return "mse", err.reshape(1), {"aux": 1}            # the first one-element tensor is the loss
flextrain.set_llm_func(lambda i: model.blocks[i], get_batch, pre_process, layer_forward, post_process, loss_fn)
engine = flextrain.initialize(model, optimizer)
got = []
for _ in data:
    results = engine.train_iteration()
    assert len(results) == 2 and results[0][0] == "mse"
    got.append(sum(float(r[1].detach()) for r in results) / 2)
engine.shutdown()
worst = max(abs(a - b) for a, b in zip(got, want))
assert worst < 2e-5, (got, want)
print("user model ok", worst)
'''


def test_stock_torch_modules_through_the_reference_style_api():
    proc = subprocess.run([sys.executable, "-c", SCRIPT % ROOT], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "user model ok" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]
