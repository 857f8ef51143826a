"""Helpers shared by the GPU parity tests."""
import torch

O_TOL = 1e-3   # relative L2, bf16 outputs vs the fp64 checker's output rounded to bf16
S_TOL = 1e-4   # relative L2, fp32 final states vs the fp64 checker


def dev(inp):
    return inp.to("cuda")


def check_o(O, o_gpu, o_ref, tol=O_TOL):
    err = O.rel_l2(o_gpu.float().cpu(), o_ref.to(torch.bfloat16).float())
    assert err <= tol, f"output rel-L2 {err:.3e} > {tol}"
    return err


def check_s(O, s_gpu, s_ref, tol=S_TOL):
    err = O.rel_l2(s_gpu.float().cpu(), s_ref)
    assert err <= tol, f"state rel-L2 {err:.3e} > {tol}"
    return err
