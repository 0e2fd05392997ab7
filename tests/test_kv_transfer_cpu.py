"""KV-transfer components on CPU: LMCache ops against index arithmetic, the pinned pool and
the point-to-point connector (PUT / PUT_ASYNC / GET, spill, NACK, missing tensor)."""
import torch

from vllm_gcu_b200.ops import ref
from vllm_gcu_b200.parallel.kv_transfer import P2PKVConnector, TensorMemoryPool, lmcache_ops


def test_multi_and_single_layer_transfer_roundtrip():
    torch.manual_seed(0)
    L, slots, W, T = 3, 40, 16, 9
    layers = [torch.randn(2, slots, W) for _ in range(L)]
    sm = torch.randperm(slots)[:T]
    sm[2] = -1
    buf = torch.zeros(2, L, T, W)
    lmcache_ops.multi_layer_kv_transfer(buf, torch.zeros(L, dtype=torch.int64), sm, "cpu", slots,
                                        True, False, layers=layers)
    for l in range(L):
        for t in range(T):
            if sm[t] >= 0:
                assert torch.equal(buf[0, l, t], layers[l][0, sm[t]])
                assert torch.equal(buf[1, l, t], layers[l][1, sm[t]])
    fresh = [torch.zeros(2, slots, W) for _ in range(L)]
    lmcache_ops.multi_layer_kv_transfer(buf, torch.zeros(L, dtype=torch.int64), sm, "cpu", slots,
                                        False, False, layers=fresh)
    for l in range(L):
        v = sm[sm >= 0]
        assert torch.equal(fresh[l][:, v], layers[l][:, v])
    one = torch.zeros(T, 2, W)
    lmcache_ops.single_layer_kv_transfer(one, layers[1][0], layers[1][1], sm, True, True)
    assert torch.equal(one[0, 1], layers[1][1, sm[0]])


def test_rerotation_equals_fresh_rotation():
    torch.manual_seed(1)
    T, H, D = 6, 2, 32
    cs = ref.make_cos_sin_cache(D, 128)
    k = torch.randn(T, H * D)
    old = torch.randint(0, 60, (T,))
    new = old + torch.randint(0, 60, (T,))
    for neox in (True, False):
        _, k_old = ref.rotary_embedding(old, k.clone(), k.clone(), D, cs, neox)
        _, k_new = ref.rotary_embedding(new, k.clone(), k.clone(), D, cs, neox)
        moved = k_old.clone()
        lmcache_ops.rotary_embedding_k_fused(old, new, moved, D, cs, neox)
        assert torch.allclose(moved, k_new, atol=1e-4)


def test_cachegen_cdf():
    x = torch.randint(0, 8, (2, 50, 5), dtype=torch.int8)
    cdf = lmcache_ops.calculate_cdf(x, 8)
    assert cdf.shape == (2, 5, 9)
    c = cdf.to(torch.int32) & 0xFFFF
    assert (c[..., 0] == 0).all() and (c[..., -1] == 65535).all()
    assert (c[..., 1:] >= c[..., :-1]).all()


def test_memory_pool_reuse():
    pool = TensorMemoryPool(4096, pin=False)
    a = pool.store(torch.arange(256, dtype=torch.float32))
    b = pool.store(torch.ones(256, dtype=torch.float32))
    assert a is not None and b is not None and a != b
    assert pool.store(torch.zeros(1024, dtype=torch.float32)) is None
    assert torch.equal(pool.load(a, (256,), torch.float32, "cpu"),
                       torch.arange(256, dtype=torch.float32))
    pool.release(a)
    pool.release(b)
    assert pool.store(torch.zeros(1000, dtype=torch.float32)) is not None


def test_p2p_connector_put_spill_nack_get():
    prod = P2PKVConnector(send_type="PUT", mem_pool_size=0)
    cons = P2PKVConnector(send_type="PUT", kv_buffer_size=1024, mem_pool_size=2048)
    try:
        t1 = torch.randn(4, 32)                       # 512 B: fits the device budget
        t2 = torch.randn(8, 32)                       # 1 KiB: spills to the pinned pool
        t3 = torch.randn(64, 32)                      # 8 KiB: nowhere to go -> NACK
        assert prod.send_tensor("r1#l0", t1, cons.addr)
        assert prod.send_tensor("r1#l1", t2, cons.addr)
        assert not prod.send_tensor("r1#l2", t3, cons.addr)
        assert torch.equal(cons.recv_tensor("r1#l0"), t1)
        assert torch.equal(cons.recv_tensor("r1#l1"), t2)
        assert cons.recv_tensor("r1#l2", timeout_s=0.2) is None   # consumer recomputes
        assert cons.stats["spilled"] == 1 and prod.stats["nack"] == 1
    finally:
        prod.close()
        cons.close()
    p2 = P2PKVConnector(send_type="GET")
    c2 = P2PKVConnector(send_type="GET")
    try:
        t = torch.randn(3, 7)
        p2.send_tensor("r9#l0", t, c2.addr)
        assert torch.equal(c2.recv_tensor("r9#l0", remote=p2.addr), t)
        assert c2.recv_tensor("missing#l0", remote=p2.addr) is None
    finally:
        p2.close()
        c2.close()
    pa = P2PKVConnector(send_type="PUT_ASYNC")
    ca = P2PKVConnector(send_type="PUT")
    try:
        t = torch.randn(5, 5)
        assert pa.send_tensor("ra#l0", t, ca.addr)
        assert torch.equal(ca.recv_tensor("ra#l0", timeout_s=10), t)
    finally:
        pa.close()
        ca.close()


def test_cachegen_codec_roundtrip_reference():
    """CacheGen arithmetic codec, host reference: decode(encode(x)) == x with the table of the
    same data and with a table from other data (symbols it never saw stay codable); the packed
    (prefix-sum) decoder reads the same streams; compressible data shrinks."""
    import torch
    from vllm_gcu_b200.parallel.kv_transfer import lmcache_ops as O
    torch.manual_seed(0)
    L, T, C, bins = 2, 5, 24, 16
    skew = torch.distributions.Categorical(torch.tensor([0.6, 0.2, 0.1] + [0.1 / 13] * 13))
    sym = skew.sample((L, T, C)).to(torch.int8)
    cdf = O.calculate_cdf(sym, bins)
    out = torch.zeros(L, T, 3 * C + 8, dtype=torch.uint8)
    lens = torch.zeros(L, T, dtype=torch.int32)
    O.encode_fast_new(cdf, sym, out, lens)
    assert int(lens.min()) > 0 and int(lens.max()) < C      # well under one byte per symbol
    dec = torch.zeros_like(sym)
    O.decode_fast_new(cdf, out, lens, dec)
    assert torch.equal(dec, sym)
    # packed layout
    flat, offs = [], [0]
    for l in range(L):
        for t in range(T):
            flat += out[l, t, :int(lens[l, t])].tolist()
            offs.append(len(flat))
    dec2 = torch.zeros_like(sym)
    O.decode_fast_prefsum(cdf, torch.tensor(flat, dtype=torch.uint8),
                          torch.tensor(offs, dtype=torch.int64), dec2)
    assert torch.equal(dec2, sym)
    # a table built from different data still round-trips
    other = O.calculate_cdf(torch.randint(0, 4, (L, T, C)).to(torch.int8), bins)
    O.encode_fast_new(other, sym, out, lens)
    dec3 = torch.zeros_like(sym)
    O.decode_fast_new(other, out, lens, dec3)
    assert torch.equal(dec3, sym)


def test_disaggregated_prefill_one_prefill_one_decode_instance():
    """1P1D: the prefill engine ships the prompt's KV through the point-to-point connector,
    the decode engine injects it, computes only the last prompt token and continues; the
    tokens equal those of a single engine.  A missing transfer falls back to local prefill."""
    import torch
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    kw = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
              num_gpu_blocks=64, dtype="float32", seed=0)
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, 32000, (37,), generator=g).tolist()
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    want = LLM("tiny-llama", **kw).generate([prompt], sp)[0].outputs[0].token_ids

    pre, dec = LLM("tiny-llama", **kw), LLM("tiny-llama", **kw)
    cp, cd = P2PKVConnector(send_type="PUT"), P2PKVConnector(send_type="PUT")
    try:
        dp = pre.engine.attach_kv_connector(cp)
        dd = dec.engine.attach_kv_connector(cd, recv_timeout_s=5.0)
        rid = pre.engine.add_request(prompt, SamplingParams(max_tokens=1, temperature=0.0,
                                                            ignore_eos=True),
                                     request_id="r-77",
                                     kv_transfer_params={"do_remote_decode": True,
                                                         "remote": cd.addr})
        first = None
        while pre.engine.has_unfinished():
            for o in pre.engine.step():
                if o.finished:
                    first = o.outputs[0].token_ids
        assert first == want[:1] and dp.stats["sent"] == 1
        dec.engine.add_request(prompt, sp, request_id="d-1",
                               kv_transfer_params={"do_remote_prefill": True, "remote": cp.addr,
                                                   "remote_request_id": rid})
        assert dd.stats["injected"] == 1
        got = None
        steps = 0
        while dec.engine.has_unfinished():
            steps += 1
            for o in dec.engine.step():
                if o.finished:
                    got = o.outputs[0].token_ids
        assert got == want
        assert dec.engine.stats["prefill_tokens"] <= 1 or steps <= 7   # no full local prefill
        # nothing was sent for this id: falls back to computing the prompt locally
        dd.recv_timeout_s = 0.2
        dec.engine.add_request(prompt, sp, request_id="d-2",
                               kv_transfer_params={"do_remote_prefill": True, "remote": cp.addr,
                                                   "remote_request_id": "missing"})
        assert dd.stats["fallback"] == 1
        got2 = None
        while dec.engine.has_unfinished():
            for o in dec.engine.step():
                if o.finished:
                    got2 = o.outputs[0].token_ids
        assert got2 == want
    finally:
        cp.close()
        cd.close()


def test_disaggregated_prefill_first_token_reuse_and_block_granular(monkeypatch):
    """The two switches of the reference's NIXL patch: with first-token reuse the decode
    instance computes no prompt token at all (it continues from the prefill instance's first
    output token); with full-KV transfer off it takes whole blocks only and recomputes the
    tail.  Both give the tokens of a single engine."""
    import torch
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    kw = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
              num_gpu_blocks=64, dtype="float32", seed=0)
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, 32000, (37,), generator=g).tolist()
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    want = LLM("tiny-llama", **kw).generate([prompt], sp)[0].outputs[0].token_ids
    monkeypatch.setenv("VLLM_B200_NIXL_ENABLE_FIRST_TOKEN_REUSE", "1")
    pre, dec = LLM("tiny-llama", **kw), LLM("tiny-llama", **kw)
    cp, cd = P2PKVConnector(send_type="PUT"), P2PKVConnector(send_type="PUT")
    try:
        pre.engine.attach_kv_connector(cp)
        dd = dec.engine.attach_kv_connector(cd, recv_timeout_s=5.0)

        def prefill(rid):
            pre.engine.add_request(prompt, SamplingParams(max_tokens=1, temperature=0.0,
                                                          ignore_eos=True), request_id=rid,
                                   kv_transfer_params={"do_remote_decode": True,
                                                       "remote": cd.addr})
            params = None
            while pre.engine.has_unfinished():
                for o in pre.engine.step():
                    if o.finished:
                        params = o.kv_transfer_params
            return params

        def decode(rid, params, max_tokens):
            dec.engine.add_request(list(prompt), SamplingParams(max_tokens=max_tokens,
                                                                temperature=0.0, ignore_eos=True),
                                   request_id=rid, kv_transfer_params=params)
            n0 = dec.engine.stats["prefill_tokens"]
            got = None
            while dec.engine.has_unfinished():
                for o in dec.engine.step():
                    if o.finished:
                        got = o.outputs[0].token_ids
            return got, dec.engine.stats["prefill_tokens"] - n0

        params = prefill("p-1")
        assert params["do_remote_prefill"] and params["remote_request_id"] == "p-1"
        assert params["first_token"] == want[0] and params["remote"] == cp.addr
        # the first token is part of the decode instance's prompt: it produces the other five
        got, _ = decode("d-1", params, 5)
        assert dd.stats["injected"] == 1 and dd.stats["first_token_reused"] == 1
        assert got == want[1:]
        # whole blocks only: 32 of 37 prompt tokens are taken, 5 are computed again
        monkeypatch.setenv("VLLM_B200_NIXL_ENABLE_FIRST_TOKEN_REUSE", "0")
        monkeypatch.setenv("VLLM_B200_NIXL_ENABLE_FULL_KV_TRANSFER", "0")
        params = prefill("p-2")
        assert params["first_token"] is None
        got, _ = decode("d-2", params, 6)
        assert got == want and dd.stats["injected"] == 2
    finally:
        cp.close()
        cd.close()


def test_connector_on_an_explicit_port_reports_its_address():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    c = P2PKVConnector(port=port)
    try:
        assert c.port == port and c.addr == f"127.0.0.1:{port}"
    finally:
        c.close()
