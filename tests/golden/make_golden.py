"""Generate the golden vectors under tests/golden/ from the reference's own PyTorch code.

Run once in a container where the reference project is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports, by file path, the reference's pure-PyTorch implementations

    build/torch28-cxx11-cu129-x86_64-linux/yamoe/reference.py   (GptOssExperts, both branches)
    torch-ext/yamoe/vendored/gpt_oss_mlp.py                     (its twin)
    torch-ext/yamoe/vendored/yamoe_ref.py                       (binned, capacity-aware)

runs them on CPU on seeded inputs, checks that they agree with each other where they
should, and writes inputs + outputs as .npz files (`subops_small.npz`: binned_gather / binned_scatter of
yamoe_ref.py for the standalone gather / scatter operators).  The only change made to the imported
code is that `yamoe_ref.sort_tokens_by_expert` is replaced by a version calling
`torch.sort(stable=True)`: the reference CUDA path sorts with a stable radix sort
(csrc/sort.cu:30) while yamoe_ref.py:40 uses torch's default sort, which is not stable on
CPU, and the capacity drop depends on that order.

The full-size README workload (T=512, H=2880, E=8, K=2, fp32) is stored as a digest: a
strided sub-sample of the reference output and fp64 row sums; its inputs are regenerated
from the seed by oracle.experts_oracle.make_readme_inputs.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import experts_oracle as orc  # noqa: E402


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build_ref(mod, inp, E, H, K, train):
    cfg = types.SimpleNamespace(intermediate_size=H, num_local_experts=E, hidden_size=H,
                                num_experts_per_tok=K)
    m = mod.GptOssExperts(cfg)
    with torch.no_grad():
        m.gate_up_proj.copy_(inp["gate_up_proj"])
        m.gate_up_proj_bias.copy_(inp["gate_up_proj_bias"])
        m.down_proj.copy_(inp["down_proj"])
        m.down_proj_bias.copy_(inp["down_proj_bias"])
    m.train(train)
    return m


def small_inputs(T, H, E, K, seed, with_grad=True):
    d = orc.make_inputs(T, H, E, K, seed=seed, weight_std=0.35, bias_std=0.5, with_grad=with_grad)
    return d


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    reference = load(os.path.join(ref_root, "build/torch28-cxx11-cu129-x86_64-linux/yamoe/reference.py"), "ref_reference")
    twin = load(os.path.join(ref_root, "torch-ext/yamoe/vendored/gpt_oss_mlp.py"), "ref_gpt_oss_mlp")
    yref = load(os.path.join(ref_root, "torch-ext/yamoe/vendored/yamoe_ref.py"), "ref_yamoe_ref")

    def stable_sort_tokens(router_indices, num_experts):
        flat = router_indices.flatten()
        sv, si = torch.sort(flat, stable=True)
        tpe = torch.bincount(sv, minlength=num_experts)
        return si, sv, torch.cumsum(tpe, 0), tpe
    yref.sort_tokens_by_expert = stable_sort_tokens

    cases = [("small_a", 40, 32, 8, 2, 1), ("small_b", 33, 48, 5, 3, 2), ("small_c", 64, 32, 16, 4, 3),
             ("small_d", 7, 32, 4, 1, 4)]
    for name, T, H, E, K, seed in cases:
        inp = small_inputs(T, H, E, K, seed)
        args = (inp["hidden_states"].view(1, T, H), inp["router_indices"], inp["routing_weights"])
        with torch.no_grad():
            out_train = build_ref(reference, inp, E, H, K, True)(*args).view(T, H)
            out_eval = build_ref(reference, inp, E, H, K, False)(*args).view(T, H)
            out_twin = build_ref(twin, inp, E, H, K, True)(*args).view(T, H)
            cap_full = T
            out_binned = yref.binned_experts_ref(args[0], inp["router_indices"], inp["routing_weights"],
                                                 inp["gate_up_proj"], inp["gate_up_proj_bias"],
                                                 inp["down_proj"], inp["down_proj_bias"], cap_full).view(T, H)
            cap_small = max(1, (T * K) // (2 * E))
            out_drop = yref.binned_experts_ref(args[0], inp["router_indices"], inp["routing_weights"],
                                               inp["gate_up_proj"], inp["gate_up_proj_bias"],
                                               inp["down_proj"], inp["down_proj_bias"], cap_small).view(T, H)
        assert torch.allclose(out_train, out_eval, rtol=1e-4, atol=1e-4)
        assert torch.allclose(out_train, out_twin, rtol=1e-5, atol=1e-5)
        assert torch.allclose(out_train, out_binned, rtol=1e-4, atol=1e-4)
        # autograd through the training branch
        m = build_ref(reference, inp, E, H, K, True)
        hs = inp["hidden_states"].clone().requires_grad_(True)
        rw = inp["routing_weights"].clone().requires_grad_(True)
        out = m(hs.view(1, T, H), inp["router_indices"], rw).view(T, H)
        (out * inp["grad_out"]).sum().backward()
        sv, si, counts, bins = orc.route_oracle(inp["router_indices"], E)
        save = {k: v.numpy() for k, v in inp.items()}
        save.update(out_train=out_train.numpy(), out_eval=out_eval.numpy(), out_drop=out_drop.numpy(),
                    cap_small=np.int64(cap_small),
                    d_hidden=hs.grad.numpy(), d_routing=rw.grad.numpy(),
                    d_wgu=m.gate_up_proj.grad.numpy(), d_bgu=m.gate_up_proj_bias.grad.numpy(),
                    d_wd=m.down_proj.grad.numpy(), d_bd=m.down_proj_bias.grad.numpy(),
                    sorted_values=sv.numpy(), sorted_indices=si.numpy(), bins=bins.numpy(),
                    dims=np.array([T, H, E, K], dtype=np.int64))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **save)
        print(name, "ok", out_train.abs().max().item())

    # gradients under a dropping capacity: autograd through binned_experts_ref (stable sort)
    drop = {}
    for name, T, H, E, K, seed in cases:
        inp = small_inputs(T, H, E, K, seed)
        cap_small = max(1, (T * K) // (2 * E))
        leaves = {k: inp[k].clone().requires_grad_(True) for k in
                  ("hidden_states", "routing_weights", "gate_up_proj", "gate_up_proj_bias", "down_proj", "down_proj_bias")}
        out = yref.binned_experts_ref(leaves["hidden_states"].view(1, T, H), inp["router_indices"],
                                      leaves["routing_weights"], leaves["gate_up_proj"], leaves["gate_up_proj_bias"],
                                      leaves["down_proj"], leaves["down_proj_bias"], cap_small).view(T, H)
        (out * inp["grad_out"]).sum().backward()
        for key, leaf in zip(("d_hidden", "d_routing", "d_wgu", "d_bgu", "d_wd", "d_bd"), leaves.values()):
            drop[f"{name}_{key}"] = leaf.grad.numpy()
        drop[f"{name}_cap"] = np.int64(cap_small)
    np.savez_compressed(os.path.join(HERE, "drop_grads.npz"), **drop)
    print("drop_grads ok")

    # whole layer (router + experts) from the vendored GptOssMLP
    T, H, E, K = 48, 32, 8, 2
    cfg = types.SimpleNamespace(intermediate_size=H, num_local_experts=E, hidden_size=H, num_experts_per_tok=K)
    gen = torch.Generator().manual_seed(7)
    mlp = twin.GptOssMLP(cfg)
    with torch.no_grad():
        for prm, std in ((mlp.router.weight, 0.5), (mlp.router.bias, 0.5), (mlp.experts.gate_up_proj, 0.35),
                         (mlp.experts.gate_up_proj_bias, 0.5), (mlp.experts.down_proj, 0.35),
                         (mlp.experts.down_proj_bias, 0.5)):
            prm.copy_(torch.randn(prm.shape, generator=gen) * std)
    x = torch.randn(2, T // 2, H, generator=gen)
    mlp.train(False)
    with torch.no_grad():
        out_mlp, scores = mlp(x)
    np.savez_compressed(os.path.join(HERE, "mlp_small.npz"), x=x.numpy(), out=out_mlp.numpy(), scores=scores.numpy(),
                        router_weight=mlp.router.weight.detach().numpy(), router_bias=mlp.router.bias.detach().numpy(),
                        gate_up_proj=mlp.experts.gate_up_proj.detach().numpy(),
                        gate_up_proj_bias=mlp.experts.gate_up_proj_bias.detach().numpy(),
                        down_proj=mlp.experts.down_proj.detach().numpy(),
                        down_proj_bias=mlp.experts.down_proj_bias.detach().numpy(),
                        dims=np.array([T, H, E, K], dtype=np.int64))
    print("mlp_small ok", out_mlp.abs().max().item())

    # the padded [E, C, H] sub-operators: binned_gather / binned_scatter of yamoe_ref.py
    T, H, E, K = 37, 24, 6, 3
    inp = small_inputs(T, H, E, K, 11, with_grad=False)
    sv, si, counts, bins = orc.route_oracle(inp["router_indices"], E)
    sub = {}
    for cap in (T, 5):
        g = yref.binned_gather(inp["hidden_states"], si, bins[:E], cap, K)
        gen = torch.Generator().manual_seed(cap)
        src = torch.randn(E, cap, H, generator=gen)
        sel = torch.gather(inp["routing_weights"], 1, inp["router_indices"]).reshape(-1)
        sc = yref.binned_scatter(src, si, sel, bins[:E], cap, K)
        sc_plain = yref.binned_scatter(src, si, None, bins[:E], cap, K)
        sub.update({f"gather_c{cap}": g.numpy(), f"src_c{cap}": src.numpy(), f"scatter_c{cap}": sc.numpy(),
                    f"scatter_plain_c{cap}": sc_plain.numpy()})
    np.savez_compressed(os.path.join(HERE, "subops_small.npz"), hidden_states=inp["hidden_states"].numpy(),
                        router_indices=inp["router_indices"].numpy(), routing_weights=inp["routing_weights"].numpy(),
                        sorted_indices=si.numpy(), bins=bins.numpy(), dims=np.array([T, H, E, K], dtype=np.int64),
                        **sub)
    print("subops_small ok")

    # README workload digest (full size, fp32, forward only)
    inp = orc.make_readme_inputs(batch=2)
    T, H, E, K = 512, 2880, 8, 2
    args = (inp["hidden_states"].view(2, 256, H), inp["router_indices"], inp["routing_weights"])
    with torch.no_grad():
        out_train = build_ref(reference, inp, E, H, K, True)(*args).reshape(T, H)
        out_eval = build_ref(reference, inp, E, H, K, False)(*args).reshape(T, H)
    sv, si, counts, bins = orc.route_oracle(inp["router_indices"], E)
    np.savez_compressed(os.path.join(HERE, "readme_digest.npz"),
                        sub_train=out_train[::16, ::45].numpy(), sub_eval=out_eval[::16, ::45].numpy(),
                        rowsum_train=out_train.double().sum(1).numpy(),
                        absmax=np.float64(out_train.abs().max().item()),
                        counts=counts.numpy(), bins=bins.numpy(),
                        sorted_indices_head=si[:64].numpy(),
                        hidden_head=inp["hidden_states"][0, :8].numpy())
    print("readme digest ok", out_train.abs().max().item(), counts.tolist())


if __name__ == "__main__":
    main()
