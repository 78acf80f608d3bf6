"""The conversation-cache policy driving the real engine's snapshot / restore calls (mk_park, mk_unpark, mk_side_begin,
mk_side_unpark, mk_side_end_park) with sequences shaped like a server's: an agent conversation, a client's title request beside
it and that request's follow-up, a second agent session, the first one coming back, an edit of its history. Checked at every step:
the store calls the policy makes, and that the cache the engine holds afterwards is bit for bit the one it should be (the state
digest of engine.cu:1438-1500 over rows and rings): the kept conversation after a side request, the parked one after it comes
back, and at the end a fresh engine that was given the final token sequence in one go."""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MARK = "<|im_start|>assistant"
LONG = "please look at this long file: " + "0123456789 " * 260  # about 2,900 tokens: longer than the q8_0 window


def render(msgs):
    text = "".join("<|im_start|>%s\n%s<|im_end|>\n" % (m["role"], m["content"]) for m in msgs)
    return [ord(c) for c in text + "<|im_start|>assistant\n"]


def user(text):
    return [{"role": "user", "content": text}]


def follow_up(msgs, reply, text="more"):
    return msgs + [{"role": "assistant", "content": reply}, {"role": "user", "content": text}]


def make_rows(torch, layers):
    """K / V rows as a function of (token, position, layer): a token table plus a position table"""
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    E = torch.randn((layers, 2, 256, 4, 256), generator=g, device="cuda")
    P = torch.randn((layers, 2, 509, 4, 256), generator=g, device="cuda") * 0.5

    def rows(tokens, pos0, layer):
        t = torch.tensor(tokens, device="cuda")
        p = (torch.arange(len(tokens), device="cuda") + pos0) % 509
        return (E[layer, 0][t] + P[layer, 0][p]).half().contiguous(), (E[layer, 1][t] + P[layer, 1][p]).half().contiguous()
    return rows


@pytest.mark.parametrize("exact", [False, True])
def test_a_servers_sequence_of_requests_through_the_policy(mk, torch_cuda, exact):
    torch = torch_cuda
    policy = importlib.import_module("qwen38-megakernel_b200.cache_policy")
    convm = importlib.import_module("qwen38-megakernel_b200.conversation")
    layers, ctx, spec, win = 2, 8192, "K*=5r,V*=6", 2048
    rows = make_rows(torch, layers)
    eng = mk.Engine(layers, ctx, spec, win, exact=exact)
    eng.store_budget(256 << 20)
    eng.store_reserve(192 << 20)  # the pinned chunks now, so that a box that will not pin that much shows here and not as "no room" later
    if eng.store_info()["allocated"] < (192 << 20):
        eng.close()
        pytest.skip("this box does not give 192 MiB of pinned host memory")
    conv = convm.KvConversation(eng, layers, rows, exact=exact)
    cache = policy.ConversationCache(conv, policy.Limits(park_mib=256, park_min=50, park_cks=2, side_max=200), tuple(ord(c) for c in MARK))
    names = lambda: [o[0] for o in conv.ops]  # noqa: E731

    def chat(msgs, reply="ab", tools=True, max_tokens=-1):
        toks = render(msgs)
        first = not any(m["role"] == "assistant" for m in msgs)
        did = convm.switch(cache, toks, (), first, max_tokens, tools)
        after_switch = eng.state_digest().copy() if eng.position() else None
        pos, how = convm.serve(cache, toks, [ord(c) for c in reply], (), tools, len(toks) - len("<|im_start|>assistant\n"))
        return did, how, after_switch

    a1, b1, s1 = user("A: " + LONG), user("B: " + LONG), user("a title please")
    # 1. the agent conversation A
    assert chat(a1)[:2] == ("none", "reset")
    seq_a, d_a = conv.sequence(), eng.state_digest().copy()
    assert eng.position() == len(seq_a) == len(render(a1)) + 2
    # 2. a client's title request runs beside it; its own conversation is parked as a side entry; A is back untouched
    assert chat(s1, tools=False)[0] == "side"
    assert names() == ["side_begin", "side_end_park"]
    assert conv.sequence() == seq_a and np.array_equal(eng.state_digest(), d_a) and not eng.side_active()
    assert [(e.side, len(e.seq)) for e in cache.parked.values()] == [(True, len(render(s1)) + 2)]
    # 3. its follow-up continues the parked side conversation, beside A again
    assert chat(follow_up(s1, "ab"), tools=False)[0] == "side-resume"
    assert names()[2:] == ["side_begin", "side_unpark", "side_end_park"]
    assert conv.sequence() == seq_a and np.array_equal(eng.state_digest(), d_a)
    assert eng.store_info()["parked"] == 1 and cache.counters["side_resumed"] == 1
    # 4. a second agent session: A is parked
    did, how, _ = chat(b1)
    assert (did, how) == ("park", "reset") and names()[-1] == "park"
    seq_b, d_b = conv.sequence(), eng.state_digest().copy()
    assert not np.array_equal(d_b, d_a)
    # 5. A's next turn: B is parked, A comes back from the host store bit for bit, then continues
    a2 = follow_up(a1, "ab", "and now the tests")
    did, how, restored = chat(a2, reply="cd")
    assert did == "unpark" and names()[-2:] == ["park", "unpark"]
    assert np.array_equal(restored, d_a)
    assert how == ("checkpoint" if exact else "append")
    assert conv.sequence() == render(a2) + [ord("c"), ord("d")]
    # 6. B's next turn: the other way round
    did, how, restored = chat(follow_up(b1, "ab", "go on"))
    assert did == "unpark" and np.array_equal(restored, d_b), "\n".join(cache.lines + [str(conv.ops), str(eng.store_info())])
    # 7. A again, with a block moved out of a later message (an edited history): nothing new is parked for it beyond the swap,
    #    the engine resumes at a checkpoint
    a3 = follow_up(a1, "ab", "and now the tests, please") + [{"role": "assistant", "content": "cd"}, {"role": "user", "content": "thanks"}]
    did, how, _ = chat(a3)
    assert did == "unpark" and how == "checkpoint"
    assert conv.sequence() == render(a3) + [ord("a"), ord("b")]
    assert cache.counters["parks"] == 4 and cache.counters["park_restores"] == 3 and eng.store_info()["parked"] == 2

    # the cache the engine holds now against a fresh engine given the final tokens in one go
    fresh = mk.Engine(layers, ctx, spec, win, exact=exact)
    ref = convm.KvConversation(fresh, layers, rows, exact=exact)
    ref.prefill(conv.sequence(), checkpoint=False)
    n = eng.position()
    assert fresh.position() == n
    if exact:
        # exact mode: every resume went through a checkpoint with its ring snapshot: identical to never having left
        assert np.array_equal(eng.state_digest(), fresh.state_digest())
    g = torch.Generator(device="cuda")
    g.manual_seed(9)
    T = 8
    for layer in range(layers):
        Q = torch.randn((T, 24, 256), generator=g, device="cuda").half()
        K, V = rows([7] * T, n, layer)
        O1 = torch.empty((T, 24, 256), dtype=torch.float32, device="cuda")
        O2 = torch.empty_like(O1)
        eng.step(layer, n, K, V, Q, O1)
        fresh.step(layer, n, K, V, Q, O2)
        eng.sync()
        fresh.sync()
        if exact:
            assert torch.equal(O1, O2)
        else:
            # the window rows behind a rewind are rebuilt from the low-bit rows (ring refill), as in the reference without MK_EXACT
            assert float((O1 - O2).abs().max()) <= 5e-2 and torch.isfinite(O1).all()
    fresh.close()
    eng.close()
