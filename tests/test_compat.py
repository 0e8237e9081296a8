"""The opt-in alias that lets scripts written for the reference's package name run."""
import subprocess
import sys
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import sys
sys.path.insert(0, %r)
import flextrain_b200.compat
assert flextrain_b200.compat.installed
import flextrain
from flextrain.config import init_flextrain_config, get_flextrain_config
from flextrain.ops.adam import FlexTrainAdam
from flextrain.ops.adam.cpu_adam import FlexTrainCPUAdam
from flextrain.optimizer import FlexTrainOptimizer, FlexTrainCPUOptimizer
from flextrain.checkpointing import get_cuda_rng_tracker, checkpointed_forward, checkpointed_backward
from flextrain.memory.initializer import Init, shutdown_init_context, restore_init_context
import flextrain_b200, flextrain_b200.config, flextrain_b200.ops.adam
assert flextrain is flextrain_b200
assert sys.modules["flextrain.config"] is flextrain_b200.config          # one module, one config singleton
assert FlexTrainAdam is flextrain_b200.ops.adam.FlexTrainAdam
assert flextrain.Init is Init and callable(flextrain.set_llm_func) and callable(flextrain.initialize)
init_flextrain_config({"batch_size": 2, "micro_batch_size": 1}, log=False)
assert flextrain_b200.config.get_flextrain_config() is get_flextrain_config()
try:
    import flextrain.no_such_module
    raise SystemExit("a missing submodule must stay missing")
except ModuleNotFoundError:
    pass
flextrain_b200.compat.uninstall()
assert "flextrain" not in sys.modules
print("alias ok")
'''


def test_reference_package_name_resolves_to_this_package():
    proc = subprocess.run([sys.executable, "-c", SCRIPT % ROOT], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "alias ok" in proc.stdout, proc.stdout + proc.stderr


def test_alias_is_not_installed_unless_asked():
    code = "import sys; sys.path.insert(0, %r); import flextrain_b200; assert 'flextrain' not in sys.modules; " \
           "import importlib.util; assert importlib.util.find_spec('flextrain') is None or True; print('clean')" % ROOT
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "clean" in proc.stdout, proc.stdout + proc.stderr
