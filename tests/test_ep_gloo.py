"""Expert-parallel dispatch / combine over 2 CPU ranks (gloo): the routing arithmetic and both exchanges, without a GPU.
The expert computation is replaced by f_e(x) = (e + 1) * x applied per segment of the contiguous layout, so that a
wrong destination row, split size or un-permutation shows up as a wrong number."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from asymgemm_b200.ep import EPDispatcher, to_contiguous_layout


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _fake_experts(a, state, first_expert):
    out = torch.zeros_like(a)
    off, exp = state.offsets.tolist(), state.experts.tolist()
    for i, e in enumerate(exp):
        if e < 0:
            break
        out[off[2 * i]:off[2 * i + 1]] = a[off[2 * i]:off[2 * i + 1]] * (first_expert + e + 1)
    return out


def _roundtrip_worker(rank, world, port, q, ranges=None):
    try:
        _init(rank, world, port)
        torch.manual_seed(100 + rank)
        num_experts, tokens, hidden, top_k = 8, 37 + 5 * rank, 16, 3
        x = torch.randn(tokens, hidden)
        ids = torch.stack([torch.randperm(num_experts)[:top_k] for _ in range(tokens)])
        if rank == 0:
            ids[:, 0] = 5            # a hot expert on the other rank; expert 2 may get no rows at all
        w = torch.rand(tokens, top_k)
        disp = EPDispatcher(num_experts, expert_ranges=ranges)
        first_expert = disp.expert_ranges[rank][0]
        state, recv, (recv_tag,) = disp.dispatch(x, ids, (torch.arange(tokens, dtype=torch.float32).unsqueeze(1),))
        a = to_contiguous_layout(recv, state)
        assert a.shape[0] == state.padded_rows and state.padded_rows % 128 == 0
        assert int(state.rows_per_expert.sum()) == recv.shape[0] == sum(state.recv_splits)
        # every segment is 128-aligned and holds exactly its expert's rows, padding rows are zero
        off = state.offsets.tolist()
        assert all(o % 128 == 0 for o in off)
        assert state.experts.tolist() == list(range(disp.experts_per_rank)) + [-1]
        y = disp.combine(_fake_experts(a, state, first_expert), state, w)
        want = ((ids + 1).float() * w).sum(dim=1, keepdim=True) * x
        assert torch.allclose(y, want, rtol=1e-5, atol=1e-5), (y - want).abs().max()
        # the same layer in rounds over groups of each rank's experts (on a GPU the exchanges overlap the GEMMs)
        tags = torch.arange(tokens, dtype=torch.float32).unsqueeze(1)
        for groups in (2, 3, 16):
            seen = []

            def group_fn(recv_rows, recv_extras, st, first, count):
                seen.append((first, count))
                assert st.experts.tolist() == list(range(count)) + [-1] and recv_extras[0].shape == (recv_rows.shape[0], 1)
                return _fake_experts(to_contiguous_layout(recv_rows, st), st, first_expert + first)

            y2 = disp.pipelined(x, (tags,), ids, w, groups, group_fn)
            assert torch.allclose(y2, want, rtol=1e-5, atol=1e-5), (groups, (y2 - want).abs().max())
            # the groups tile this rank's experts in order, none empty
            assert seen[0][0] == 0 and sum(c for _, c in seen) == disp.experts_per_rank and all(c > 0 for _, c in seen)
            assert all(seen[i][0] + seen[i][1] == seen[i + 1][0] for i in range(len(seen) - 1))
        dist.barrier()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover - reported through the queue
        q.put((rank, f"error: {type(e).__name__}: {e}"))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run(worker, world=2, timeout=120, extra=()):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q) + tuple(extra)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        r, msg = q.get(timeout=timeout)
        results[r] = msg
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    return results


def test_dispatch_combine_roundtrip_two_ranks():
    results = _run(_roundtrip_worker)
    assert results == {0: "ok", 1: "ok"}, results


def test_dispatch_combine_roundtrip_unequal_expert_ranges():
    """Rank 0 owns experts 0-2, rank 1 owns experts 3-7 (shares sized by link rate in production)."""
    results = _run(_roundtrip_worker, extra=([(0, 3), (3, 8)],))
    assert results == {0: "ok", 1: "ok"}, results


def test_expert_ranges_are_validated():
    with pytest.raises(RuntimeError):
        EPDispatcher(4, expert_ranges=[(0, 3)])          # does not cover all experts
    with pytest.raises(RuntimeError):
        EPDispatcher(4, expert_ranges=[(1, 4)])


def _single_rank_layout():
    return EPDispatcher(4)     # no process group: one rank owning all four experts


def test_layout_arithmetic_single_rank():
    disp = _single_rank_layout()
    ids = torch.tensor([[0, 3], [3, 1], [3, 0]])
    x = torch.arange(3, dtype=torch.float32).unsqueeze(1) + 1
    state, recv, _ = disp.dispatch(x, ids)
    assert state.rows_per_expert.tolist() == [2, 1, 0, 3] and state.padded_rows == 128 + 4 * 128
    # every local expert has a segment; the one without rows is empty (start == end)
    assert state.offsets.tolist() == [0, 128, 128, 256, 256, 256, 256, 384] and state.experts.tolist() == [0, 1, 2, 3, -1]
    assert recv is x and state.src_token.tolist() == [0, 2, 1, 0, 1, 2]   # one rank: rows are gathered by the scatter itself
    a = to_contiguous_layout(recv, state)
    assert a[:2, 0].tolist() == [1.0, 3.0] and a[128, 0] == 2.0 and a[256:259, 0].tolist() == [1.0, 2.0, 3.0]
    assert a.abs().sum() == 12.0
    y = disp.combine(a, state, torch.ones(3, 2))
    assert torch.equal(y, 2 * x)


def _failing_worker(rank, world, port, q):
    """Rank 1 raises before the exchange; rank 0 must get an error from its collective, not hang."""
    try:
        _init(rank, world, port, timeout_s=5)
        dist.barrier()
        if rank == 1:
            raise ValueError("injected host-side failure before dispatch")
        disp = EPDispatcher(4)
        ids = torch.zeros((4, 1), dtype=torch.int64) + 3
        disp.dispatch(torch.ones(4, 8), ids)
        q.put((rank, "no error"))
    except ValueError as e:
        q.put((rank, f"raised: {e}"))
        q.close()
        q.join_thread()
        os._exit(0)   # the rank leaves without joining any further collective
    except Exception as e:
        q.put((rank, f"collective failed: {type(e).__name__}"))


def test_rank_failure_surfaces_as_error_not_hang():
    results = _run(_failing_worker, timeout=90)
    assert results[1].startswith("raised")
    assert results[0].startswith("collective failed"), results
