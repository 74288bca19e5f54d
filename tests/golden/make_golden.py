"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own oracle code on CPU.

Usage (in a container that has the reference checkout):
    python tests/golden/make_golden.py <path to the reference checkout>

The reference's test module cannot be imported as a whole (it imports the CUDA extension and runs
a CUDA test at import time), so this script parses it with ``ast`` and executes only the function
definitions it needs, unmodified:
    test/test_flex_block_attn.py : create_mask, torch_attn_test, generate_tensor
    benchmark/utils/utils.py     : create_sparse_mask, create_torch_mask, torch_attn
Inputs are drawn by the reference's ``generate_tensor`` (mean 0.1, std 10 magnitudes) from
torch.manual_seed(0) on CPU, rounded to bf16 (what the kernels see) and stored as bf16 bit
patterns; the expected O and the gradients w.r.t. Q, K, V are what the reference's oracle
(``F.scaled_dot_product_attention`` with the dense token mask + autograd) returns in fp32.
The committed .npz files are what the tests read; the reference itself is not needed at test time.
"""
from __future__ import annotations

import ast
import random
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_functions(path: Path, names):
    tree = ast.parse(path.read_text())
    keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in keep}
    if missing:
        raise RuntimeError(f"{path}: missing {missing}")
    ns = {"torch": torch, "np": np, "F": torch.nn.functional, "random": random}
    exec(compile(ast.Module(body=keep, type_ignores=[]), str(path), "exec"), ns)
    return [ns[n] for n in names]


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)


def run_case(fns, seq_len, heads, q_block, kv_block):
    create_mask, torch_attn_test, generate_tensor = fns
    torch.manual_seed(0)
    shape = (1, heads, seq_len, 128)
    mk = lambda: generate_tensor(shape, 1e-1, 10, torch.float32, "cpu").to(torch.bfloat16).float()
    Q, K, V, dO = mk(), mk(), mk(), mk()
    Q.requires_grad_(), K.requires_grad_(), V.requires_grad_()
    import contextlib, io
    with contextlib.redirect_stdout(io.StringIO()):
        torch_mask, block_mask = create_mask(Q, q_block, kv_block)
    o = torch_attn_test(Q, K, V, torch_mask)
    o.backward(dO)
    return dict(
        q=bf16_bits(Q.detach()), k=bf16_bits(K.detach()), v=bf16_bits(V.detach()), do=bf16_bits(dO),
        block_mask=block_mask.numpy(), q_block=np.int32(q_block), kv_block=np.int32(kv_block),
        o=o.detach().numpy(), dq=Q.grad.numpy(), dk=K.grad.numpy(), dv=V.grad.numpy(),
    )


def run_bench_style_case(fns, seq_len, block, keep):
    """Mask and oracle exactly as the reference's benchmark harness builds them
    (utils.py:94-119,132-138); selected blocks drawn like generate_selected_blocks (:69-83)."""
    create_sparse_mask, create_torch_mask, torch_attn = fns
    torch.manual_seed(1)
    random.seed(1)
    shape = (1, 1, seq_len, 128)
    mk = lambda: torch.randn(shape).to(torch.bfloat16).float()
    Q, K, V, dO = mk(), mk(), mk(), mk()
    Q.requires_grad_(), K.requires_grad_(), V.requires_grad_()
    nb = seq_len // block
    selected = [(i, j) for i in range(nb) for j in random.sample(range(nb), int(nb * keep))]
    block_mask = create_sparse_mask(Q, block, selected)
    torch_mask = create_torch_mask(Q, block, selected)
    o = torch_attn(Q, K, V, torch_mask)
    o.backward(dO)
    return dict(
        q=bf16_bits(Q.detach()), k=bf16_bits(K.detach()), v=bf16_bits(V.detach()), do=bf16_bits(dO),
        block_mask=block_mask.numpy(), q_block=np.int32(block), kv_block=np.int32(block),
        o=o.detach().numpy(), dq=Q.grad.numpy(), dk=K.grad.numpy(), dv=V.grad.numpy(),
    )


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
    ref = Path(sys.argv[1])
    test_fns = load_functions(ref / "test" / "test_flex_block_attn.py",
                              ["create_mask", "torch_attn_test", "generate_tensor"])
    bench_fns = load_functions(ref / "benchmark" / "utils" / "utils.py",
                               ["create_sparse_mask", "create_torch_mask", "torch_attn"])
    cases = {
        # the reference's import-time smoke case (test_flex_block_attn.py:142)
        "ref_test_s128_h1_q16_k64": run_case(test_fns, 128, 1, 16, 64),
        # two points of the reference's parametrised block-size grid (:66-71) at shorter seq_len, long
        # enough that kv-block column 4 of the mask rule (:25) exists and every row attends
        "ref_test_s384_h1_q16_k64": run_case(test_fns, 384, 1, 16, 64),
        "ref_test_s640_h1_q32_k128": run_case(test_fns, 640, 1, 32, 128),
        # the benchmark harness' mask / oracle path with equal 128 blocks
        "ref_bench_s512_b128_keep50": run_bench_style_case(bench_fns, 512, 128, 0.5),
    }
    for name, d in cases.items():
        np.savez(HERE / f"{name}.npz", **d)
        print(name, {k: getattr(v, "shape", v) for k, v in d.items()})


if __name__ == "__main__":
    main()
