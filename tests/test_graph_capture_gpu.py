"""CUDA-graph capture of the two recurrences: the reference's kernel functions are graph-capturable (its GEMM benchmark
replays them from a graph), so the replayed calls here must reproduce the eagerly launched ones bit for bit."""
import pytest
import torch

from avelang_b200 import synth

pytestmark = pytest.mark.gpu


def test_decode_step_replays_from_a_graph(built_lib):
    from avelang_b200 import gdn
    inp = synth.config2(n_seqs=32, n_slots=64, Hk=2, Hv=4).to("cuda")
    pool_eager, pool_graph = inp.state_pool.clone(), inp.state_pool.clone()
    out_eager = torch.empty_like(inp.v)
    out_graph = torch.empty_like(inp.v)
    call = lambda pool, out: gdn.fused_recurrent_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, initial_state=pool,
                                                                  state_indices=inp.state_indices, out=out)
    call(pool_eager.clone(), out_eager)  # first call outside capture: library handles, status word
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call(pool_graph, out_graph)
    for _ in range(3):
        graph.replay()
        call(pool_eager, out_eager)
    torch.cuda.synchronize()
    assert torch.equal(out_graph, out_eager) and torch.equal(pool_graph, pool_eager)


def test_prefill_replays_from_a_graph(built_lib):
    """One long sequence: the call forks onto the library's helper streams (range-overlapped schedule) and joins back,
    which a capture has to follow."""
    from avelang_b200 import gdn
    inp = synth.make_inputs(1, 2048 + 37, 2, 4, 128, 128, seed=5, with_z=True).to("cuda")
    run = lambda out: gdn.chunk_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, output_final_state=True, z=inp.z, out=out)
    o_eager = torch.empty_like(inp.v)
    _, s_eager = run(o_eager)  # also creates the helper streams and events outside capture
    torch.cuda.synchronize()
    o_graph = torch.empty_like(inp.v)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        _, s_graph = run(o_graph)
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(o_graph, o_eager) and torch.equal(s_graph, s_eager)
