"""Child process of tests/test_gpu_engine.py::test_tensor_transfer_over_cuda_ipc: rebuilds a tensor from the request
dict it reads from a file, checks it, writes a reply tensor into the shared memory and exits."""
import pickle
import sys

import torch

sys.path.insert(0, sys.argv[2])
from multimodal_training_b200.runtime.tensor_transfer import receive_tensor  # noqa: E402

req = pickle.load(open(sys.argv[1], "rb"))
torch.cuda.set_device(0)
t = receive_tensor(req)
assert t.is_cuda and tuple(t.shape) == tuple(req["shape"])
total = float(t.double().sum())
t.mul_(2)                                   # the producer sees this: same physical memory
torch.cuda.synchronize()
print(f"SUM {total!r}")
