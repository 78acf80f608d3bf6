"""Token-level view of the KV engine for the conversation-cache policy (cache_policy.ConversationCache): the engine protocol the
reference's server speaks to its Engine (server/mk_engine.py: sequence, committed, checkpoints, park .. side_drop), on top of this
package's Engine, which knows positions and rows only. The tokens of the live conversation and of every parked one are kept here on
the host, next to the ids the engine's store hands out; the rows of a token come from the caller (`rows(tokens, pos0, layer)`
-> (K, V) fp16 [n][4][256] on the device: in a server, the model's projections; in the tests, rows derived from the token ids).

request(cache, tokens, ...) is one request of the reference's request loop (mk_server.py load_prompt + generate, as far as the cache
is concerned): cache_switch, resume where resume_point says, prefill the rest of the prompt, checkpoint at its end, append the reply,
then side_finish / debris_finish."""
from .cache_policy import ConversationCache  # noqa: F401  (re-exported for callers that import this module only)


class KvConversation:
    side_keep = True   # the library has side_end_park / side_unpark
    ck_pins = False    # no pinned checkpoints in this path

    def __init__(self, eng, layers, rows, exact=False, block=4096):
        self.eng, self.layers, self.rows, self.exact, self.block = eng, layers, rows, bool(exact), block
        self.seq = []          # tokens of the engine's sequence
        self.entries = {}      # id -> tokens of a parked conversation
        self.kept = None       # tokens of the sequence a side request keeps aside
        self.ops = []          # (name, ...) of every store call made, for the caller's log and the tests

    # ---- what the policy reads ----
    def sequence(self):
        return list(self.seq)

    def committed(self):
        return self.eng.position()

    def checkpoints(self):
        return self.eng.checkpoints()

    def store_info(self):
        d = dict(self.eng.store_info())
        d["last_ms"], d["side_ms"], d["side_park_ms"] = d["last_us"] / 1e3, d["side_us"] / 1e3, d["side_park_us"] / 1e3
        return d

    def kv_sizes(self):
        s = self.eng.kv_sizes()
        return s["per_token"], s["rings"], s["state"], s["checkpoint"]

    def park_need(self, k):
        return self.eng.park_need(k)

    # ---- the sequence ----
    def prefill(self, tokens, checkpoint=True):
        """rows of `tokens` appended at the end of the sequence, every layer; a checkpoint at the end of a prompt"""
        pos0 = len(self.seq)
        for a in range(0, len(tokens), self.block):
            part = tokens[a:a + self.block]
            for layer in range(self.layers):
                K, V = self.rows(part, pos0 + a, layer)
                self.eng.append(layer, pos0 + a, K, V)
        self.seq.extend(tokens)
        self.eng.commit(len(self.seq))
        if checkpoint and tokens:
            self.eng.checkpoint()

    def resume(self, pos, how):
        """the engine's sequence cut back to `pos` the way resume_point chose"""
        if how == "append":
            if pos < len(self.seq):
                self.eng.truncate(pos)
        elif how == "checkpoint":
            if not self.eng.rewind_to(pos):
                raise RuntimeError("rewind_to: no checkpoint at %d" % pos)
        else:
            # (cut to nothing rather than the engine's reset: that would also end a side request and drop what it keeps aside)
            if self.eng.position() > 0:
                self.eng.truncate(0)
            pos = 0
        del self.seq[pos:]

    # ---- the store ----
    def park(self, k):
        pid = self.eng.park(k)
        self.ops.append(("park", pid, len(self.seq)))
        if pid is None or pid == 0:
            return None
        self.entries[pid] = list(self.seq)
        return pid

    def unpark(self, pid):
        self.eng.unpark(pid)
        self.seq = self.entries.pop(pid)
        self.ops.append(("unpark", pid, len(self.seq)))

    def park_drop(self, pid):
        self.entries.pop(pid, None)
        self.ops.append(("park_drop", pid))
        return self.eng.park_drop(pid)

    def side_begin(self):
        ok = self.eng.side_begin()
        self.ops.append(("side_begin", ok))
        if ok:
            self.kept, self.seq = self.seq, []
        return ok

    def side_active(self):
        return self.eng.side_active()

    def side_unpark(self, pid):
        ok = self.eng.side_unpark(pid)
        self.ops.append(("side_unpark", pid, ok))
        if ok:
            self.seq = self.entries.pop(pid)
        return ok

    def side_end(self):
        back = self.eng.side_end()
        self.ops.append(("side_end", back))
        self.seq, self.kept = (self.kept if back else []), None
        return back

    def side_end_park(self, k):
        own = list(self.seq)
        back, pid = self.eng.side_end_park(k)
        self.ops.append(("side_end_park", pid or None, back))
        if pid:
            self.entries[pid] = own
        if back:
            self.seq = self.kept
        self.kept = None
        return back, (pid or None)

    def side_drop(self):
        self.eng.side_drop()
        self.ops.append(("side_drop",))
        self.seq, self.kept = [], None


def switch(cache, tokens, spans=(), first_turn=False, max_tokens=-1, tools=True):
    """the first half of a request: the cache's decision between replies; returns what cache_switch did"""
    cache.rid += 1
    return cache.cache_switch(tokens, list(spans), first_turn, max_tokens, tools)


def serve(cache, tokens, reply, spans=(), tools=True, gen=None, answer_tokens=None):
    """the second half: resume where resume_point says, prefill the rest of the prompt (a checkpoint at its end), append the reply,
    finish a side request. Returns (resume position, how)."""
    conv = cache.eng
    _, _, pos, how = cache.resume_point(conv.sequence(), conv.committed(), conv.checkpoints(), cache.img_spans, tokens, list(spans))
    conv.resume(pos, how)
    conv.prefill(tokens[pos:])
    cache.img_spans = list(spans)
    cache.live_gen = len(tokens) - 1 if gen is None else gen
    cache.live_tools = bool(tools)
    if cache.side is None:
        cache.live_low = cache.next_low
    cache.side_ready = True
    conv.prefill(list(reply), checkpoint=False)
    cache.answer_tokens = len(reply) if answer_tokens is None else answer_tokens
    cache.side_finish()
    cache.debris_finish(True)
    return pos, how


def request(cache, tokens, reply, spans=(), first_turn=False, max_tokens=-1, tools=True, gen=None, answer_tokens=None):
    """One request against cache.eng (a KvConversation): returns (what cache_switch did, resume position, how). `reply`: the tokens
    the model answers with (appended after the prompt); gen: where the prompt's generation prompt starts (default: its last token)."""
    did = switch(cache, tokens, spans, first_turn, max_tokens, tools)
    pos, how = serve(cache, tokens, reply, spans, tools, gen, answer_tokens)
    return did, pos, how
