"""The conversation-cache policy that calls the snapshot / restore API: which conversation the engine holds between two
replies, which ones wait in the pinned host store, and which go first when the store is full.

Mirrors the reference's server/mk_srv_cache.py:29-332 (class CacheMixin: resume_point, cache_switch, first_reply, store_update,
make_room, evict, park_live, unpark, side_start, side_finish, debris_finish; class Parked :7-16; the constants :19-26) rule for
rule, as a class of its own instead of a mixin of an HTTP server: the caller hands in the engine, the limits and, per request, the
prompt's tokens. The decisions are host logic only; every byte moves through the engine's calls (park, unpark, park_drop,
side_begin, side_unpark, side_end, side_end_park, side_drop), which this package's Engine maps onto mk_park .. mk_side_drop.

Engine protocol (what the reference's server expects of its Engine, server/mk_engine.py): sequence() -> cached tokens,
committed() -> positions whose state cannot be cut back without a checkpoint, checkpoints() -> positions, exact (bool),
park_need(k), park(k) -> id | None, unpark(id), park_drop(id), store_info() -> dict(used, allocated, last_bytes, last_ms, side_ms
[, side_park_bytes, side_park_ms]), kv_sizes() -> (per token, rings, state, checkpoint) bytes, side_begin() -> bool,
side_unpark(id) -> bool, side_end() -> bool, side_end_park(k) -> (bool, id | None), side_drop(), side_active(); optional:
side_keep (bool), ck_pins (bool) with pinned()."""
import time
from dataclasses import dataclass, field

# server/mk_srv_cache.py:19-26
SIDE_STORE_MIB = 1024     # the store of side requests when parking is off
SIDE_REPLY_MAX = 1024     # with parking on, a request with tools is a side request only if its reply is capped at this
SIDE_REPLY_ROOM = 8192    # rows of store room taken for a reply without a cap
SIDE_PARK_CKS = 1         # checkpoints parked with a side request's own conversation
SIDE_KEEP_MAX = 4         # side requests' conversations kept at most
SUMMARY_ANSWER_MIN = 256  # an answer this long (thinking aside) to a long prompt without tools is taken for a summary


@dataclass
class Limits:
    """the server's command line, as far as the cache reads it (mk_server.py --park-mib / --park-min / --park-cks / --side-max)"""
    park_mib: int = 0      # host memory for parked conversations; 0: parking off
    park_min: int = 1024   # conversations shorter than this are not worth a copy
    park_cks: int = 2      # newest checkpoints parked with a conversation
    side_max: int = 0      # longest prompt that may run as a side request; 0: side requests off


@dataclass
class Parked:
    """one entry of the host store as the policy sees it (mk_srv_cache.py:7-16). side: a side request's own conversation; low:
    likely never continued; both go before the others. gen: where its generation prompt starts (-1: unknown)"""
    id: int
    seq: list
    cks: list
    committed: int
    img_spans: list
    gen: int
    nbytes: int
    side: bool = False
    low: bool = False
    tools: object = None
    pins: tuple = ()
    t: float = field(default_factory=time.time)


@dataclass
class Live:
    """what the policy remembers about the engine's own conversation: its image spans, where its generation prompt starts (-1:
    unknown), whether its last request had tools (None: unknown) and why it has low priority ("": it has not)"""
    spans: list = field(default_factory=list)
    gen: int = -1
    tools: object = None
    low: str = ""


def common_prefix(a, b):
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


def _mib(n):
    return "%.1f MiB" % (n / 1048576.0)


class ConversationCache:
    """State and decisions of the host cache for one engine. The caller's request loop:

        cache.cache_switch(tokens, spans, first_turn, max_tokens, tools)   # may park / unpark / begin a side request
        match, cut, pos, how = cache.resume_point(eng.sequence(), eng.committed(), eng.checkpoints(), cache.img_spans, tokens, spans)
        ... rewind or reset the engine to pos as `how` says, prefill tokens[pos:], decode the reply ...
        cache.side_ready = True once the prompt is processed; cache.answer_tokens = tokens of the answer
        cache.side_finish(); cache.debris_finish(replied)
    """

    def __init__(self, eng, limits, asst_marker=(), log=None):
        self.eng, self.args = eng, limits
        self.asst_marker = tuple(asst_marker)
        self.parked = {} if (limits.park_mib > 0 or limits.side_max > 0) else None  # id -> Parked, least recently parked first
        self.store_mib = limits.park_mib if limits.park_mib > 0 else SIDE_STORE_MIB
        self.live = Live()
        self.side, self.side_ready, self.answer_tokens = None, False, 0
        self.cache_pre, self.next_low, self.debris = "", "", None
        self.counters, self.store_gauge, self.rid = {}, (), 0
        self.lines = []
        self._log = log

    # ---- the marks of the live conversation under the names the reference's server uses ----
    img_spans = property(lambda self: self.live.spans, lambda self, v: setattr(self.live, "spans", v))
    live_gen = property(lambda self: self.live.gen, lambda self, v: setattr(self.live, "gen", v))
    live_tools = property(lambda self: self.live.tools, lambda self, v: setattr(self.live, "tools", v))
    live_low = property(lambda self: self.live.low, lambda self, v: setattr(self.live, "low", v))

    # ---- small helpers ----
    def log(self, text):
        line = "#%d %s" % (self.rid, text)
        self.lines.append(line)
        if self._log:
            self._log(line)

    def count(self, **kw):
        for k, v in kw.items():
            self.counters[k] = self.counters.get(k, 0) + v

    def side_keep(self):
        """mk_srv_cache.py:30-34: a side request's own conversation is parked after it"""
        lim = self.args
        if self.parked is None or lim.side_max <= 0 or lim.park_mib <= 0:
            return False
        return bool(getattr(self.eng, "side_keep", False))

    def _budget(self):
        return self.args.park_mib << 20

    def _used(self):
        return self.eng.store_info()["used"]

    # ---- where a prompt would resume on a cached sequence (mk_srv_cache.py:37-53) ----
    def resume_point(self, seq, committed, cks, cached_spans, toks, spans):
        """Returns (tokens shared with the cache, position of the image span that shortened that or None, where the engine
        would resume, how: 'append', 'checkpoint' or 'reset'). The last prompt token is always processed again; an image span
        present on one side only cuts the prefix at its start; past the committed length the cached sequence continues by
        appending (not in exact mode), before it only a checkpoint can be resumed."""
        match = min(common_prefix(seq, toks), len(toks) - 1)
        pos, cut = match, None
        for p, _, _ in set(spans) ^ set(cached_spans):
            if p < pos:
                pos = cut = p
        if seq and pos >= committed and not self.eng.exact:
            return match, cut, pos, "append"
        ck = max((p for p in cks if 0 < p <= pos), default=0)
        return match, cut, ck, ("checkpoint" if ck else "reset")

    def _resume_on(self, e, toks, spans):
        return self.resume_point(e.seq, e.committed, e.cks, e.img_spans, toks, spans)

    # ---- the switch between replies (mk_srv_cache.py:55-131) ----
    def cache_switch(self, toks, spans, first_turn, max_tokens=-1, tools=True):
        """Returns what was done, for the caller's log and the tests: 'side-resume', 'side', 'unpark', 'unpark+park', 'edit',
        'park', 'none'."""
        self.cache_pre = self.next_low = ""
        self.debris = None
        eng, a, seq = self.eng, self.args, self.eng.sequence()
        live = self.resume_point(seq, eng.committed(), eng.checkpoints(), self.live.spans, toks, spans)
        lost = len(seq) - live[2]                                  # cached positions the plain path would throw away
        continues = 0 <= self.live.gen <= live[0]                  # the prompt reaches the live one's generation prompt
        bounded = 0 < max_tokens <= SIDE_REPLY_MAX
        side_ok = (a.side_max > 0 and len(toks) <= a.side_max and not continues and lost >= max(2 * len(toks), a.park_min)
                   and (a.park_mib <= 0 or not tools or bounded))

        # 1. a one-shot that continues a side request's own parked conversation: beside the live one again
        if side_ok and self.side_keep() and self.parked:
            pick = None
            for e in self.parked.values():
                if e.side and e.gen >= 0:
                    r = self._resume_on(e, toks, spans)
                    if r[0] >= e.gen and r[2] > live[2] and (pick is None or r[2] > pick[1][2]):
                        pick = (e, r)
            if pick:
                self.side_start(seq, len(toks), max_tokens, resume=pick[0])
                return "side-resume"

        # 2. a parked conversation that the prompt continues at least park_min further than the live one: they swap
        if a.park_mib > 0 and self.parked:
            pick = None
            for e in self.parked.values():
                r = self._resume_on(e, toks, spans)
                if r[2] >= live[2] + a.park_min and (pick is None or r[2] > pick[1][2]):
                    pick = (e, r)
            if pick:
                e, r = pick
                self.park_live(seq, "another conversation came back", keep=e.id, low=self.live.low)
                self.unpark(e)
                shares_only_pinned_head = r[2] in e.pins and r[0] < e.gen
                if not shares_only_pinned_head:
                    return "unpark"
                # a new session on the same system prompt: the restored conversation goes back to the store whole
                again_low = "it was parked with low priority" if e.low else ""
                self.park_live(eng.sequence(), "a new session reuses its system prompt", low=again_low)
                return "unpark+park"

        # 3. a first turn - or, with parking on, a request without tools that would displace a conversation with tools - runs
        #    beside the live conversation
        beside_tools = bool(self.live.tools) and not tools and a.park_mib > 0
        if side_ok and (first_turn or beside_tools):
            summary_like = not tools and len(toks) >= a.park_min and a.park_mib > 0
            self.side_start(seq, len(toks), max_tokens,
                            after="replaced right after a summary request beside it" if summary_like else "")
            return "side"

        # 4. the request discards at least park_min cached positions: the live conversation is parked first, unless the prompt
        #    is that same conversation with its later history edited
        if a.park_mib > 0 and not continues and lost >= a.park_min:
            k = self.first_reply(toks)
            same_start = k is not None and k + len(self.asst_marker) <= live[0]
            if same_start:
                self.log("not parked: the prompt is the cached conversation with its history edited (it matches %d of the %d cached "
                         "tokens, past its first reply at %d)" % (live[0], len(seq), k))
                return "edit"
            debris = "replaced by a request without tools" if (self.live.tools and not tools) else ""
            provisional = bool(debris) and not self.live.low
            entry = self.park_live(seq, "a new conversation", low=self.live.low or debris, provisional=provisional)
            if provisional:
                self.debris = entry
            if debris:
                self.next_low = "the conversation of a request without tools that replaced one with tools"
            return "park"
        return "none"

    def first_reply(self, toks):
        """position of the prompt's first assistant marker (mk_srv_cache.py:133-147), or None"""
        m = self.asst_marker
        if not m:
            return None
        n = len(m)
        for k in range(0, len(toks) - n + 1):
            if toks[k] == m[0] and tuple(toks[k:k + n]) == m:
                return k
        return None

    # ---- the store's bookkeeping (mk_srv_cache.py:149-176) ----
    def store_update(self):
        info = self.eng.store_info()
        ps = list(self.parked.values()) if self.parked else []
        self.store_gauge = (len(ps), info["used"], info["allocated"], tuple(len(e.seq) for e in ps),
                            sum(1 for e in ps if e.side), sum(1 for e in ps if e.low))
        return info

    def make_room(self, need, budget, keep=None, side_only=False):
        """Evicts until `need` more bytes fit in `budget`: side requests' conversations and low-priority ones first, then (unless
        side_only) the others, each tier least recently parked first, never `keep`. False: it does not fit."""
        while self._used() + need > budget:
            victim = None
            for pid, e in self.parked.items():
                if pid != keep and (e.side or e.low):
                    victim = pid
                    break
            if victim is None and not side_only:
                victim = next((pid for pid in self.parked if pid != keep), None)
            if victim is None:
                return False
            e = self.parked[victim]
            tier = "a side request's" if e.side else "low priority" if e.low else "normal priority"
            self.evict(victim, "least recently parked, %s, to make room" % tier)
        return True

    def evict(self, pid, why):
        self.eng.park_drop(pid)
        e = self.parked.pop(pid)
        self.store_update()
        self.count(park_evictions=1)
        self.log("evicted the parked conversation of %d tokens (%s; %s)" % (len(e.seq), _mib(e.nbytes), why))

    # ---- park / unpark (mk_srv_cache.py:178-235) ----
    def park_live(self, seq, why, keep=None, low="", provisional=False):
        """Snapshot of the live conversation into the store; returns its entry or None. A low-priority one (unless the mark is
        provisional) only takes room that side and low-priority entries can give: it never evicts a normal one."""
        eng, a = self.eng, self.args
        if len(seq) < a.park_min:
            return None
        need, budget = eng.park_need(a.park_cks), self._budget()
        if need > budget:
            self.log("not parked: the cached %d tokens need %s of host memory (limit %d MiB)" % (len(seq), _mib(need), a.park_mib))
            return None
        if low and not provisional:
            giveable = sum(e.nbytes for pid, e in self.parked.items() if pid != keep and (e.side or e.low))
            if need > budget - self._used() + giveable or not self.make_room(need, budget, keep, side_only=True):
                self.log("not parked: the cached %d tokens (%s) have low priority (%s) and do not fit without evicting a conversation "
                         "of normal priority" % (len(seq), _mib(need), low))
                return None
        else:
            self.make_room(need, budget, keep)
        pins, cks = [], []
        if a.park_cks > 0:  # what the engine parks: the newest park_cks checkpoints and the pinned ones
            if getattr(eng, "ck_pins", False):
                pins = list(eng.pinned())
            newest = sorted(eng.checkpoints())[-a.park_cks:]
            cks = sorted(set(newest).union(pins))
        pid = eng.park(a.park_cks)
        if pid is None:
            self.log("not parked: no room in the host store for the cached %d tokens (%s)" % (len(seq), _mib(need)))
            return None
        e = Parked(pid, list(seq), cks, eng.committed(), self.live.spans, self.live.gen, need, low=bool(low), tools=self.live.tools,
                   pins=tuple(pins))
        self.parked[pid] = e
        info = self.store_update()
        self.count(parks=1)
        self.log("parked the cached conversation (%s%s): %d tokens, %s | %d parked, %s of %d MiB" % (
            why, ", low priority: " + low if low else "", len(seq), _mib(info.get("last_bytes", 0)), len(self.parked),
            _mib(info["used"]), a.park_mib))
        return e

    def unpark(self, e):
        """the engine becomes parked conversation e; its entry is freed (also when the engine fails: then the error goes on)"""
        failed = None
        try:
            self.eng.unpark(e.id)
        except RuntimeError as err:
            failed = err
        self.parked.pop(e.id, None)
        if failed is not None:
            self.eng.park_drop(e.id)  # (the entry goes too, with its host memory)
            self.store_update()
            raise failed
        self.live = Live(e.img_spans, e.gen, e.tools, "")
        self.store_update()
        self.count(park_restores=1)
        self.cache_pre = "restored a parked conversation (%d tokens); " % len(e.seq)
        self.log("restored the parked conversation of %d tokens | %d parked" % (len(e.seq), len(self.parked)))

    # ---- side requests (mk_srv_cache.py:237-317) ----
    def side_room(self, cached, n, max_tokens):
        """store bytes a side request may take: the recurrent state and rings of the kept sequence, the rows its prompt and reply
        overwrite (the reply's cap, else SIDE_REPLY_ROOM rows), and two checkpoint blocks"""
        per_token, rings, state, ck = self._sizes()
        reply = min(max_tokens, SIDE_REPLY_ROOM) if max_tokens > 0 else SIDE_REPLY_ROOM
        return state + rings + per_token * min(cached, n + reply) + 2 * ck

    def _sizes(self):
        s = self.eng.kv_sizes()
        if isinstance(s, dict):
            return s["per_token"], s["rings"], s["state"], s["checkpoint"]
        return tuple(s)

    def side_start(self, seq, n, max_tokens=-1, resume=None, after=""):
        eng = self.eng
        self.make_room(self.side_room(len(seq), n, max_tokens), self.store_mib << 20, keep=resume.id if resume else None)
        if not eng.side_begin():
            self.log("side request: no room in the host store: the cached %d tokens are not kept" % len(seq))
            return
        self.side = (len(seq), self.live, after)  # the kept conversation's marks come back with it
        self.live = Live(self.live.spans, self.live.gen, self.live.tools, self.live.low)
        self.side_ready = False
        self.count(side_requests=1)
        self.cache_pre = "side request: the cached %d tokens are kept aside; " % len(seq)
        if resume is None:
            return
        if not eng.side_unpark(resume.id):
            self.log("side request: no room in the host store to continue its parked conversation of %d tokens" % len(resume.seq))
            return
        del self.parked[resume.id]
        self.live.spans, self.live.gen, self.live.tools = resume.img_spans, resume.gen, resume.tools
        self.store_update()
        self.count(side_resumed=1)
        self.cache_pre += "its parked conversation (%d tokens) restored; " % len(resume.seq)

    def _side_conversation_to_park(self):
        """what the engine holds at the end of a side request, if it is worth parking (side_keep(), its prompt was processed and a
        checkpoint exists to resume from), with room made for it among side and low-priority entries only: (fields of its Parked
        entry or None, whether it fits)"""
        eng = self.eng
        if not (self.side_keep() and self.side_ready and eng.checkpoints()):
            return None, True
        kept_sides = [pid for pid, e in self.parked.items() if e.side]  # least recently parked first
        for pid in kept_sides[:max(0, len(kept_sides) - SIDE_KEEP_MAX + 1)]:
            self.evict(pid, "the oldest of %d kept side request conversations" % SIDE_KEEP_MAX)
        nbytes = eng.park_need(SIDE_PARK_CKS)
        own = dict(seq=list(eng.sequence()), cks=sorted(eng.checkpoints())[-SIDE_PARK_CKS:], committed=eng.committed(),
                   img_spans=self.live.spans, gen=self.live.gen, nbytes=nbytes)
        fits = nbytes <= self._budget() and self.make_room(nbytes, self._budget(), side_only=True)
        return own, fits

    def side_finish(self):
        """Ends a side request, also a failed one or one whose client left (mk_srv_cache.py:267-317). Three outcomes: the kept
        conversation is the engine's again (its marks with it; the side request's own conversation parked before, if
        _side_conversation_to_park says so); the store ran full while the side request's conversation was being parked, so that one
        stays the engine's; or nothing is left and the next request prefills in full."""
        if self.side is None:
            return
        n_kept, kept_marks, after = self.side
        self.side = None
        eng = self.eng
        back, pid, own, fits = False, None, None, True
        try:
            if eng.side_active():
                own, fits = self._side_conversation_to_park()
                if own is not None and fits:
                    back, pid = eng.side_end_park(SIDE_PARK_CKS)
                else:
                    back = eng.side_end()
        except RuntimeError as err:
            self.log("side request: %s" % err)
            eng.side_drop()
            own = None
        if pid:
            self.parked[pid] = Parked(pid, side=True, tools=self.live.tools, **own)
            self.count(side_kept=1)
        self.store_update()
        if back:
            summary = bool(after) and self.answer_tokens >= SUMMARY_ANSWER_MIN
            self.live = Live(kept_marks.spans, kept_marks.gen, kept_marks.tools, after if summary else kept_marks.low)
            note = ""
            if pid:
                note = "; its own conversation (%d tokens) parked" % len(own["seq"])
            elif own is not None:
                note = "; its own conversation was not parked (no room in the host store)"
            self.log("side request done: the cached %d tokens are back%s" % (n_kept, note))
            return
        self.count(side_dropped=1)
        if own is not None and fits:
            # side_end_park lost the kept sequence; the side request's conversation stays the engine's, with its marks
            self.log("side request: the cached %d tokens were dropped (the host store ran full): the side request's own conversation "
                     "(%d tokens) stays cached" % (n_kept, len(own["seq"])))
            return
        self.live = Live()
        self.log("side request: the cached %d tokens were dropped (the host store ran full, or an engine error): the next request "
                 "prefills its prompt in full" % n_kept)

    # ---- a provisional low-priority mark (mk_srv_cache.py:319-332) ----
    def debris_finish(self, replied):
        """The conversation with tools that a request without tools replaced was parked with a provisional low-priority mark;
        a reply shorter than a summary's takes the mark back (a title or tags task quoted it). The mark stays after a long
        answer and without a reply."""
        entry = self.debris
        self.debris = None
        if entry is None or not replied:
            return
        if self.answer_tokens >= SUMMARY_ANSWER_MIN or self.parked.get(entry.id) is not entry:
            return
        e = entry
        e.low = False
        self.store_update()
        self.log("the parked conversation of %d tokens keeps normal priority: the request answered in %d tokens (< %d: not a summary)"
                 % (len(e.seq), self.answer_tokens, SUMMARY_ANSWER_MIN))
