"""The conversation-cache policy (qwen38-megakernel_b200/cache_policy.py) against a fake engine, no GPU: the cases of the
reference's tests/test_cache_policy.py and tests/test_engine_side.py (which requests run as side requests, which edits of a
conversation's history park nothing, which parked conversations have low priority, who is evicted first), stated at the policy's
own interface instead of through an HTTP server: the sequence of store calls the engine sees is what both assert."""
import importlib

import pytest

mk_policy = importlib.import_module("qwen38-megakernel_b200.cache_policy")
mk_conv = importlib.import_module("qwen38-megakernel_b200.conversation")

MARK = "<|im_start|>assistant"
LONG = "please look at this long file: " + "0123456789 " * 40  # (well over park_min tokens)


def render(msgs, gen=True):
    """one token per character; the last '<' starts the generation prompt"""
    text = "".join("<|im_start|>%s\n%s<|im_end|>\n" % (m["role"], m["content"]) for m in msgs)
    return [ord(c) for c in text + ("<|im_start|>assistant\n" if gen else "")]


def user(text):
    return [{"role": "user", "content": text}]


class FakeEngine:
    """the store's bookkeeping without any rows: every call is recorded in ops"""
    PT, STATE, RINGS, CK = 512, 4096, 2048, 1024
    side_keep = True

    def __init__(self, budget_mib, exact=False):
        self.budget, self.exact = budget_mib << 20, exact
        self.seq, self.cks, self.entries, self.kept, self.ops, self.next_id = [], [], {}, None, [], 1
        self.side_ok, self.last_bytes, self.fail_unpark = True, 0, False

    # what the policy reads
    def sequence(self):
        return list(self.seq)

    def committed(self):
        return len(self.seq)

    def checkpoints(self):
        return list(self.cks)

    def kv_sizes(self):
        return self.PT, self.RINGS, self.STATE, self.CK

    def park_need(self, k):
        return self.STATE + self.RINGS + self.PT * len(self.seq) + self.CK * min(k, len(self.cks))

    def store_info(self):
        used = sum(e[2] for e in self.entries.values())
        if self.kept is not None:
            used += self.STATE + self.PT * min(len(self.kept[0]), 1024)
        return dict(used=used, allocated=used, last_bytes=self.last_bytes, last_ms=0.0, side_ms=0.0)

    # the sequence
    def prefill(self, tokens, checkpoint=True):
        self.seq.extend(tokens)
        if checkpoint and tokens and len(self.seq) not in self.cks:
            self.cks.append(len(self.seq))

    def resume(self, pos, how):
        if how == "reset":
            pos = 0
        del self.seq[pos:]
        self.cks = [c for c in self.cks if c <= pos]

    # the store
    def park(self, k):
        need = self.park_need(k)
        if not self.seq or self.store_info()["used"] + need > self.budget:
            self.ops.append(("park", None))
            return None
        pid, self.next_id = self.next_id, self.next_id + 1
        self.entries[pid] = (list(self.seq), list(self.cks), need)
        self.last_bytes = need
        self.ops.append(("park", pid))
        return pid

    def unpark(self, pid):
        if self.fail_unpark:
            raise RuntimeError("unpark: copy failed")
        self.seq, self.cks, _ = self.entries.pop(pid)
        self.ops.append(("unpark", pid))

    def park_drop(self, pid):
        self.ops.append(("park_drop", pid))
        return self.entries.pop(pid, None) is not None

    def side_begin(self):
        if self.budget == 0:
            self.ops.append(("side_begin", False))
            return False
        self.kept, self.seq, self.cks = (self.seq, self.cks), [], []
        self.ops.append(("side_begin", True))
        return True

    def side_active(self):
        return self.kept is not None

    def side_unpark(self, pid):
        assert self.kept is not None and not self.seq
        self.seq, self.cks, _ = self.entries.pop(pid)
        self.ops.append(("side_unpark", pid))
        return True

    def side_end(self):
        (self.seq, self.cks), self.kept = self.kept, None
        self.ops.append(("side_end",))
        return True

    def side_end_park(self, k):
        if not self.side_ok:  # the store ran full during the side request: the kept sequence is lost
            self.kept = None
            self.ops.append(("side_end_park", None, False))
            return False, None
        pid = self.park(k) if self.seq else None
        (self.seq, self.cks), self.kept = self.kept, None
        self.ops.append(("side_end_park", pid, True))
        return True, pid

    def side_drop(self):
        self.kept, self.seq, self.cks = None, [], []
        self.ops.append(("side_drop",))


def serve(park_mib=4, side_max=200, park_min=50, park_cks=2, exact=False, marker=MARK):
    eng = FakeEngine(park_mib if park_mib > 0 else mk_policy.SIDE_STORE_MIB, exact)
    cache = mk_policy.ConversationCache(eng, mk_policy.Limits(park_mib, park_min, park_cks, side_max), tuple(ord(c) for c in marker))
    return eng, cache


def chat(cache, msgs, reply="ab", tools=True, max_tokens=-1, answer_tokens=None):
    toks = render(msgs)
    first_turn = not any(m["role"] == "assistant" for m in msgs)
    gen = len(toks) - len("<|im_start|>assistant\n")
    did, _, _ = mk_conv.request(cache, toks, [ord(c) for c in reply], first_turn=first_turn, max_tokens=max_tokens, tools=tools,
                                gen=gen, answer_tokens=answer_tokens)
    return did, reply


def follow_up(msgs, reply, text="more"):
    return msgs + [{"role": "assistant", "content": reply}, {"role": "user", "content": text}]


def names(eng):
    return [o[0] for o in eng.ops]


# ---- resume_point (mk_srv_cache.py:37-53) ----

def test_resume_point_table():
    eng, cache = serve()
    seq = list(range(100))
    rp = cache.resume_point
    assert rp(seq, 100, [40, 80], [], seq + [7, 8], []) == (100, None, 100, "append")
    assert rp(seq, 100, [40, 80], [], seq[:90] + [7, 8], []) == (90, None, 80, "checkpoint")   # before committed: a checkpoint
    assert rp(seq, 100, [40, 80], [], seq[:30] + [7], []) == (30, None, 0, "reset")
    assert rp(seq, 100, [40, 80], [], seq, []) == (99, None, 80, "checkpoint")                 # the last token is processed again
    assert rp(seq, 60, [40], [], seq[:70] + [7], []) == (70, None, 70, "append")               # past committed: cut and append
    assert rp([], 0, [], [], [1, 2, 3], []) == (0, None, 0, "reset")
    # an image span on one side only cuts the prefix at its start
    assert rp(seq, 100, [40, 80], [(50, 4, "h")], seq + [7], []) == (100, 50, 40, "checkpoint")
    assert rp(seq, 100, [40, 80], [(50, 4, "h")], seq + [7], [(50, 4, "h")]) == (100, None, 100, "append")
    eng.exact = True  # exact mode: never by appending
    assert rp(seq, 100, [40, 80], [], seq + [7, 8], []) == (100, None, 80, "checkpoint")


# ---- which requests run beside the live conversation (test_cache_policy.py SideRuleTests) ----

ONE_SHOTS = {
    "session name, no max_tokens": ([{"role": "system", "content": "Generate a short title."}, {"role": "user", "content": "fix it"}], {}),
    "title, max_tokens 4096": ([{"role": "system", "content": "Session title."}, {"role": "user", "content": "hi"}], {"max_tokens": 4096}),
    "title, max_tokens 32768": (user("Generate a title for: hi"), {"max_tokens": 32768}),
    "tags, one user message": (user("### Task: tags for the chat"), {}),
}


@pytest.mark.parametrize("name", sorted(ONE_SHOTS))
def test_one_shots_without_tools_are_side_requests_whatever_their_max_tokens(name):
    msgs, kw = ONE_SHOTS[name]
    eng, cache = serve()
    chat(cache, user(LONG))
    kept = list(eng.seq)
    did, _ = chat(cache, msgs, tools=False, **kw)
    assert did == "side"
    assert names(eng) == ["side_begin", "park", "side_end_park"]
    assert eng.seq == kept                                    # the long conversation is back
    assert [(e.side, e.low) for e in cache.parked.values()] == [(True, False)]
    assert any("side request done" in l for l in cache.lines) and not any("parked the cached conversation" in l for l in cache.lines)


def test_an_agent_session_first_turn_parks_the_live_conversation():
    for kw in ({"max_tokens": 32000}, {}, {"max_tokens": 4096}):
        eng, cache = serve()
        chat(cache, user(LONG))
        did, _ = chat(cache, user("new task"), tools=True, **kw)
        assert (did, names(eng)) == ("park", ["park"]), kw
        assert any("parked the cached conversation (a new conversation)" in l for l in cache.lines)
    eng, cache = serve()  # with tools and a bounded reply: a side request
    chat(cache, user(LONG))
    assert chat(cache, user("new task"), tools=True, max_tokens=8)[0] == "side"
    assert names(eng) == ["side_begin", "park", "side_end_park"]


def test_a_chat_without_tools_continues_beside_the_live_conversation():
    eng, cache = serve()
    chat(cache, user(LONG))
    kept = list(eng.seq)
    c1 = user("hello there")
    did1, r1 = chat(cache, c1, tools=False)
    n_side = len(eng.entries[1][0])
    did2, _ = chat(cache, follow_up(c1, r1), tools=False)  # no max_tokens: continues as a side request
    assert (did1, did2) == ("side", "side-resume")
    assert names(eng) == ["side_begin", "park", "side_end_park", "side_begin", "side_unpark", "park", "side_end_park"]
    assert eng.ops[4] == ("side_unpark", 1)
    assert eng.seq == kept
    assert cache.counters == {"side_requests": 2, "side_kept": 2, "side_resumed": 1}
    assert len(list(cache.parked.values())[0].seq) > n_side  # the follow-up's conversation replaced the first turn's


def test_a_different_prompt_does_not_take_a_side_conversation():
    eng, cache = serve()
    chat(cache, user(LONG))
    chat(cache, user("a title please"), tools=False, max_tokens=4)
    chat(cache, user("a title for this one"), tools=False, max_tokens=4)
    assert [n for n in names(eng) if n.startswith("side")] == ["side_begin", "side_end_park"] * 2
    assert len(eng.entries) == 2


def test_side_requests_off_or_parking_off():
    eng, cache = serve(side_max=0)              # no side requests: the one-shot parks the live conversation
    chat(cache, user(LONG))
    assert chat(cache, user("fix it"), tools=False)[0] == "park" and names(eng) == ["park"]
    eng, cache = serve(park_mib=0)              # parking off: every short first turn is a side request, nothing is kept
    chat(cache, user(LONG))
    assert chat(cache, user("a new task"), tools=True)[0] == "side"
    assert names(eng) == ["side_begin", "side_end"]
    eng, cache = serve(park_mib=0)              # ... and a later turn is no side request
    chat(cache, user(LONG))
    c1 = user("hello there")
    assert chat(cache, follow_up(c1, "ab"), tools=False)[0] == "none" and eng.ops == []


def test_the_store_room_a_side_request_takes_follows_its_max_tokens(monkeypatch):
    monkeypatch.setattr(mk_policy, "SIDE_REPLY_ROOM", 100)
    for kw, reply in (({"max_tokens": 40}, 40), ({}, 100), ({"max_tokens": 32768}, 100)):
        eng, cache = serve()
        needs = []
        make_room = cache.make_room
        cache.make_room = lambda need, budget, keep=None, side_only=False: (needs.append(need), make_room(need, budget, keep, side_only))[1]
        chat(cache, user(LONG))
        cached = len(eng.seq)
        chat(cache, user("a title please"), tools=False, **kw)
        prompt = len(render(user("a title please")))
        assert prompt + reply < cached
        assert needs[0] == eng.STATE + eng.RINGS + eng.PT * (prompt + reply) + 2 * eng.CK, kw


# ---- edited history (test_cache_policy.py EditedHistoryTests) ----

SYS = {"role": "system", "content": "You are an agent. " * 3}
CATALOG = " <reminder>memory catalog: " + "entry " * 12 + "</reminder>"


def turn(*texts):
    msgs = [SYS]
    for i, t in enumerate(texts):
        msgs.append({"role": t[0], "content": t[1]} if isinstance(t, tuple) else {"role": "user" if i % 2 == 0 else "assistant", "content": t})
    return msgs


def run_pair(first, second, tools=True, marker=MARK):
    eng, cache = serve(side_max=0, marker=marker)
    chat(cache, first, tools=tools)
    did, _ = chat(cache, second, tools=tools)
    return did, names(eng), cache


def test_a_block_moved_out_of_a_later_message_parks_nothing():
    first = turn("fix the bug", "done, run tests?", "yes please" + CATALOG)
    second = turn("fix the bug", "done, run tests?", "yes please", "ab", "thanks" + CATALOG)
    did, ops, cache = run_pair(first, second)
    assert (did, ops) == ("edit", [])
    assert any("history edited" in l for l in cache.lines)


def test_cleared_tool_results_park_nothing():
    result = "file contents " * 8
    first = turn("read a and b", "<tool_call>read a</tool_call>", ("tool", result), "<tool_call>read b", ("tool", result), "both read",
                 "now summarize")
    second = turn("read a and b", "<tool_call>read a</tool_call>", ("tool", "[cleared]"), "<tool_call>read b", ("tool", result),
                  "both read", "now summarize", "ab", "and more")
    assert run_pair(first, second)[:2] == ("edit", [])


def test_an_edit_after_the_first_reply_parks_nothing_an_edit_of_the_first_message_parks():
    first = turn("tell me about cats", "cats are mammals " * 4, "and dogs? " * 6)
    assert run_pair(first, turn("tell me about cats", "cats are mammals " * 4, "and birds?"), tools=False)[:2] == ("edit", [])
    did, ops, cache = run_pair(first, turn("tell me about whales", "cats are mammals " * 4, "and dogs? " * 6), tools=False)
    assert (did, ops) == ("park", ["park"])
    assert any("parked the cached conversation (a new conversation)" in l for l in cache.lines)


def test_a_new_session_of_the_same_harness_still_parks_the_cached_one():
    head = "Working directory context: " + "x" * 60 + "\n"
    first = turn(head + "task A", "<tool_call>ls</tool_call>", ("tool", "a.py b.py"), "ok", "next step")
    for second in (turn(head + "task B"), turn(head + "task B", "<tool_call>ls</tool_call>", ("tool", "c.py"), "ok", "go on")):
        assert run_pair(first, second)[:2] == ("park", ["park"])


def test_without_the_role_tokens_every_divergence_parks():
    first = turn("fix the bug", "done, run tests?", "yes please" + CATALOG)
    second = turn("fix the bug", "done, run tests?", "yes please", "ab", "thanks" + CATALOG)
    assert run_pair(first, second, marker="")[:2] == ("park", ["park"])


# ---- low priority: summaries and what they replace (test_cache_policy.py DebrisTests) ----

def compaction(cache, task, summary_msgs):
    """an agent conversation (tools), its summary request (no tools, an answer of a summary's length), the compacted conversation"""
    chat(cache, user(task + LONG), tools=True)
    _, r = chat(cache, summary_msgs, reply="w" * (mk_policy.SUMMARY_ANSWER_MIN + 8), tools=False)
    chat(cache, user("Summary: " + r + " go on"), tools=True)


def test_a_summary_and_the_conversation_it_replaced_are_parked_with_low_priority():
    eng, cache = serve()
    summary = "Summarize this conversation for a continuation: " + "the user asked to read files. " * 6
    compaction(cache, "A: ", [{"role": "system", "content": "You summarize."}, {"role": "user", "content": summary}])
    text = "\n".join(cache.lines)
    assert "(a new conversation, low priority: replaced by a request without tools)" in text
    assert "(a new conversation, low priority: the conversation of a request without tools that replaced one with tools)" in text
    assert "keeps normal priority" not in text
    assert [e.low for e in cache.parked.values()] == [True, True]
    assert cache.store_gauge[0] == 2 and cache.store_gauge[5] == 2


def test_a_long_one_shot_with_a_short_answer_leaves_the_replaced_conversation_at_normal_priority():
    eng, cache = serve()
    chat(cache, user("T: " + LONG), tools=True)
    # a title task quoting the chat, longer than side_max, thinking first: its answer is 15 tokens of 293
    chat(cache, user("### Task: a title for the chat. " + LONG), reply="h" * 278 + "w" * 15, tools=False, max_tokens=1000, answer_tokens=15)
    assert [e.low for e in cache.parked.values()] == [False]
    assert any("keeps normal priority: the request answered in 15 tokens" in l for l in cache.lines)
    # without a reply (an error, the client left) the mark stays
    eng, cache = serve()
    chat(cache, user("T: " + LONG), tools=True)
    cache.rid += 1
    assert cache.cache_switch(render(user("### Task: a title. " + LONG)), [], True, 1000, False) == "park"
    cache.debris_finish(False)
    assert [e.low for e in cache.parked.values()] == [True]


def test_a_low_priority_conversation_evicts_no_conversation_of_normal_priority():
    eng, cache = serve(park_mib=1)
    eng.PT = 1400                   # (room for one long conversation)
    chat(cache, user("O: " + LONG), tools=True)
    chat(cache, user("T: " + LONG), tools=True)          # parks O (normal priority)
    assert [e.low for e in cache.parked.values()] == [False]
    per_conv = list(cache.parked.values())[0].nbytes
    assert 2 * per_conv > (1 << 20)                       # (a second one does not fit beside it)
    cache.live_low = "a test"                             # the live conversation has low priority: it may not push O out
    cache.rid += 1
    assert cache.park_live(eng.sequence(), "a new conversation", low=cache.live_low) is None
    assert any("do not fit without evicting a conversation of normal priority" in l for l in cache.lines)
    assert len(cache.parked) == 1 and "park_drop" not in names(eng)
    # a normal one does push it out
    assert cache.park_live(eng.sequence(), "a new conversation") is not None
    assert names(eng)[-2:] == ["park_drop", "park"] and cache.counters["park_evictions"] == 1


def test_side_and_low_entries_go_first_least_recently_parked_first():
    eng, cache = serve(park_mib=64)
    P = mk_policy.Parked
    for pid, (side, low) in enumerate([(False, False), (True, False), (False, True), (False, False)], start=1):
        eng.entries[pid] = ([1] * 100, [], 1000)
        cache.parked[pid] = P(pid, [1] * 100, [], 100, [], -1, 1000, side=side, low=low)
    assert cache.make_room(64 << 20, 64 << 20, keep=3, side_only=True) is False   # only the side entry may go (3 is kept)
    assert [o for o in eng.ops] == [("park_drop", 2)]
    assert cache.make_room((64 << 20) - 1500, 64 << 20) is True                    # then the low one, then the oldest normal one
    assert [o[1] for o in eng.ops] == [2, 3, 1] and list(cache.parked) == [4]


def test_at_most_four_side_conversations_are_kept():
    eng, cache = serve(park_mib=64)
    chat(cache, user(LONG))
    for i in range(6):
        chat(cache, user("a title for chat number %d please" % i), tools=False, max_tokens=4)
    sides = [e for e in cache.parked.values() if e.side]
    assert len(sides) == mk_policy.SIDE_KEEP_MAX and cache.counters["park_evictions"] == 2
    assert [e.id for e in sides] == [3, 4, 5, 6]                                  # the oldest went


# ---- a parked conversation comes back (mk_srv_cache.py:86-99) ----

def test_another_conversation_comes_back_and_the_live_one_takes_its_place():
    eng, cache = serve()
    a1, b1 = user("A: " + LONG), user("B: " + LONG)
    _, ra = chat(cache, a1)
    chat(cache, b1)                                   # parks A
    n_a = len(eng.entries[1][0])
    did, _ = chat(cache, follow_up(a1, ra))           # A continues: B is parked, A restored
    assert did == "unpark" and names(eng) == ["park", "park", "unpark"]
    assert eng.ops[2] == ("unpark", 1) and list(cache.parked) == [2]
    assert eng.seq[:n_a] == render(a1) + [ord(c) for c in ra]
    assert cache.counters["park_restores"] == 1 and cache.cache_pre.startswith("restored a parked conversation (")


def test_a_failed_unpark_frees_the_entry_and_raises():
    eng, cache = serve()
    a1 = user("A: " + LONG)
    _, ra = chat(cache, a1)
    chat(cache, user("B: " + LONG))
    eng.fail_unpark = True
    with pytest.raises(RuntimeError):
        chat(cache, follow_up(a1, ra))
    assert 1 not in cache.parked and ("park_drop", 1) in eng.ops


def test_a_side_request_that_lost_the_kept_sequence():
    eng, cache = serve()
    chat(cache, user(LONG))
    eng.side_ok = False                                # the store runs full during the side request
    chat(cache, user("a title please"), tools=False)
    assert eng.ops[-1] == ("side_end_park", None, False)
    assert cache.counters["side_dropped"] == 1 and cache.live_gen >= 0  # the side request's conversation stays the engine's
    assert any("stays cached" in l for l in cache.lines)
    # an engine error during side_end: everything is dropped, the next request prefills in full
    eng, cache = serve()
    chat(cache, user(LONG))

    def boom(k):
        raise RuntimeError("side_end_park: copy failed")
    eng.side_end_park = boom
    chat(cache, user("a title please"), tools=False)
    assert eng.ops[-1] == ("side_drop",) and (cache.live_gen, cache.live_tools, cache.img_spans) == (-1, None, [])
