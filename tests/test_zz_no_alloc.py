"""The allocation-free merge entry point against the ordinary one.

phx_topk_merge_static exists for hosts that cannot let this library allocate device memory (a
custom-call handler inside a compiler-managed step, a server whose memory pool is fully pre-sized).
Its scratch is a fixed array inside the library, shared by every call, so the test calls it twice in a
row with different inputs: the second result must not be coloured by what the first left behind.
Collected last on purpose, so a run that stops at the first failure has already run everything else."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _lists(torch, P, B, k, seed):
    """Per-shard top-k lists as the scan produces them: bf16-valued scores (many ties), unique global
    ids, each list sorted by (score desc, id asc)."""
    rng = np.random.default_rng(seed)
    sc = np.empty((P, B, k), np.float32); ids = np.empty((P, B, k), np.int64)
    for p in range(P):
        for b in range(B):
            s = torch.from_numpy(rng.standard_normal(k).astype(np.float32)).to(torch.bfloat16).float().numpy()
            i = rng.choice(1_000_000, size=k, replace=False).astype(np.int64) + p * 1_000_000
            order = np.lexsort((i, -s.astype(np.float64)))
            sc[p, b], ids[p, b] = s[order], i[order]
    return sc, ids


def test_static_merge_matches_allocating_merge_twice_in_a_row():
    import torch
    from x_algorithm_b200.retrieval import CorpusShard, merge_topk_static, merge_topk_static_status
    from x_algorithm_b200 import PhoenixError
    sh = CorpusShard(4096, 64, max_queries=16, max_k=128)      # only its merge entry point is used
    for call, (P, B, k, seed) in enumerate([(4, 16, 100, 1), (3, 9, 128, 2)]):
        sc, ids = _lists(torch, P, B, k, seed)
        d_sc, d_ids = torch.from_numpy(sc).cuda(), torch.from_numpy(ids).cuda()
        want_s = torch.empty((B, k), dtype=torch.float32, device="cuda"); want_i = torch.empty((B, k), dtype=torch.int64, device="cuda")
        got_s = torch.full((B, k), float("nan"), dtype=torch.float32, device="cuda"); got_i = torch.full((B, k), -7, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        sh.merge_device(d_sc, d_ids, P, B, k, want_s, want_i)
        sh.sync()
        free_before = torch.cuda.mem_get_info()[0]
        merge_topk_static(d_sc, d_ids, P, B, k, got_s, got_i)
        torch.cuda.synchronize()
        # the property in the entry point's name: the device's free memory is the same after the call as before it
        # (cudaMemGetInfo; the first call has already resolved the scratch array's address, which allocates nothing)
        assert torch.cuda.mem_get_info()[0] == free_before, f"call {call}: device memory was allocated"
        assert merge_topk_static_status() == 0
        np.testing.assert_array_equal(got_i.cpu().numpy(), want_i.cpu().numpy(), err_msg=f"call {call}")
        np.testing.assert_array_equal(got_s.cpu().numpy(), want_s.cpu().numpy(), err_msg=f"call {call}")
        # and both agree with the definition: (score desc, id asc) over the union
        flat_s = sc.transpose(1, 0, 2).reshape(B, -1); flat_i = ids.transpose(1, 0, 2).reshape(B, -1)
        for b in range(B):
            order = np.lexsort((flat_i[b], -flat_s[b].astype(np.float64)))[:k]
            np.testing.assert_array_equal(got_i[b].cpu().numpy(), flat_i[b][order])
    # lists shorter than k: empty slots (id -1) sort last and come back as (-inf, -1); an id that does not fit the key's
    # 32 row bits is left out and flagged in the status word
    P, B, k = 2, 3, 8
    sc = np.zeros((P, B, k), np.float32); ids = np.full((P, B, k), -1, np.int64)
    sc[:, :, :3] = np.array([0.75, 0.5, 0.25], np.float32); ids[0, :, :3] = [7, 8, 9]; ids[1, :, :3] = [4, 5, 6]
    ids[1, 2, 0] = 1 << 33
    got_s = torch.empty((B, k), dtype=torch.float32, device="cuda"); got_i = torch.empty((B, k), dtype=torch.int64, device="cuda")
    merge_topk_static(torch.from_numpy(sc).cuda(), torch.from_numpy(ids).cuda(), P, B, k, got_s, got_i)
    assert merge_topk_static_status() == 4
    gi, gs = got_i.cpu().numpy(), got_s.cpu().numpy()
    np.testing.assert_array_equal(gi[0], [4, 7, 5, 8, 6, 9, -1, -1])
    np.testing.assert_array_equal(gi[2], [7, 5, 8, 6, 9, -1, -1, -1])
    assert np.isneginf(gs[0, 6:]).all() and np.isneginf(gs[2, 5:]).all()
    # beyond the built-in scratch: refused with a clear error, nothing launched
    with pytest.raises(PhoenixError) as ei:
        merge_topk_static(d_sc, d_ids, 4096, 1024, 1024, got_s, got_i)
    assert ei.value.status == 5 and "exceeds the built-in scratch" in ei.value.message
    sh.close()
