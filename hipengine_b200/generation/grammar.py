"""Request-owned grammar constraints.

Two parts, as in the reference (``hipengine/generation/grammar.py``): (1) a generator that turns the JSON-schema
parameter blocks of OpenAI tool definitions into a Lark-syntax grammar for the Qwen XML tool-call format
(``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``), and (2) a matcher
that masks logits token by token.  The matcher delegates to ``llguidance`` (``LLMatcher`` / ``LLTokenizer``) when
that package is importable; in images without it ``grammar_available()`` is False and requests carrying a grammar
are refused before generation with ``unsupported_parameter`` (the server and ``SamplingParams`` check this), so a
constraint is never silently dropped.  The generator is pure Python and always available: the tool-call result
policy uses the same schema walk to validate arguments after generation.
"""
from __future__ import annotations

import json
import re
from typing import Any, Dict, List, Mapping, Optional, Sequence

_NAME_OK = re.compile(r"^[A-Za-z_][A-Za-z0-9_\-\.]*$")


def grammar_available() -> bool:
    try:
        import llguidance  # noqa: F401
        return True
    except Exception:
        return False


def _lit(s: str) -> str:
    return json.dumps(s)


def _value_rule(schema: Mapping[str, Any], name: str, rules: Dict[str, str]) -> str:
    """Adds rules for one parameter value and returns the rule name.  Scalars are written bare inside the
    <parameter> element; objects and arrays as JSON."""
    t = schema.get("type")
    if "enum" in schema:
        rules[name] = " | ".join(_lit(v if isinstance(v, str) else json.dumps(v)) for v in schema["enum"])
    elif t == "integer":
        rules[name] = "/-?(0|[1-9][0-9]*)/"
    elif t == "number":
        rules[name] = "/-?(0|[1-9][0-9]*)(\\.[0-9]+)?([eE][+-]?[0-9]+)?/"
    elif t == "boolean":
        rules[name] = '"true" | "false"'
    elif t == "string":
        rules[name] = "/[^<]*/"                      # any text up to the closing tag
    elif t in ("object", "array"):
        rules[name] = "json_value"
        rules.setdefault("json_value", 'json_object | json_array | json_string | json_number | "true" | "false" | "null"')
        rules.setdefault("json_object", '"{" [json_pair ("," json_pair)*] "}"')
        rules.setdefault("json_pair", 'json_string ":" json_value')
        rules.setdefault("json_array", '"[" [json_value ("," json_value)*] "]"')
        rules.setdefault("json_string", '/"([^"\\\\]|\\\\.)*"/')
        rules.setdefault("json_number", "/-?(0|[1-9][0-9]*)(\\.[0-9]+)?([eE][+-]?[0-9]+)?/")
    else:
        rules[name] = "/[^<]*/"
    return name


def tool_call_grammar(tools: Sequence[Mapping[str, Any]], allow_text_before: bool = True,
                      parallel: bool = True, only: Optional[str] = None) -> str:
    """Lark grammar accepting zero or more XML tool calls to the given functions (optionally after free text).

    Required parameters must appear, in the order of the schema's ``properties``; optional ones may be omitted.
    ``only`` restricts the grammar to one function name (``tool_choice`` naming a function)."""
    rules: Dict[str, str] = {}
    fn_rules: List[str] = []
    for ti, tool in enumerate(tools):
        fn = tool.get("function", tool)
        fname = fn.get("name", "")
        if not _NAME_OK.match(fname):
            raise ValueError(f"tool name {fname!r} cannot be expressed in the tool-call grammar")
        if only is not None and fname != only:
            continue
        params = fn.get("parameters") or {}
        props = params.get("properties") or {}
        required = set(params.get("required") or [])
        parts: List[str] = []
        for pi, (key, sch) in enumerate(props.items()):
            if not _NAME_OK.match(key):
                raise ValueError(f"parameter name {key!r} cannot be expressed in the tool-call grammar")
            vr = _value_rule(sch or {}, f"v_{ti}_{pi}", rules)
            pr = f"p_{ti}_{pi}"
            rules[pr] = f'{_lit("<parameter=" + key + ">")} ws {vr} ws "</parameter>" ws'
            parts.append(pr if key in required else f"[{pr}]")
        body = " ".join(parts) if parts else ""
        rules[f"f_{ti}"] = f'{_lit("<function=" + fname + ">")} ws {body} "</function>"'.replace("  ", " ")
        fn_rules.append(f"f_{ti}")
    if not fn_rules:
        raise ValueError("no tool matches the requested tool choice")
    rules["call"] = '"<tool_call>" ws (' + " | ".join(fn_rules) + ') ws "</tool_call>"'
    many = "call (ws call)*" if parallel else "call"
    start = f"[text] {many}" if allow_text_before else many
    lines = [f"start: {start}", "text: /[^<]+/", "ws: /[ \\t\\n]*/"]
    for k in sorted(rules):
        lines.append(f"{k}: {rules[k]}")
    return "\n".join(lines) + "\n"


class GrammarMatcher:
    """Token-level matcher over an ``llguidance`` grammar.  Only constructible when the package is present."""

    def __init__(self, lark_grammar: str, vocab: Sequence[bytes], eos_token_id: int):
        if not grammar_available():
            raise RuntimeError("grammar constraints need the llguidance package, which is not installed")
        import llguidance
        self._ll = llguidance
        self.tokenizer = llguidance.LLTokenizer(llguidance.TokenizerWrapper(
            _VocabAdapter(vocab, eos_token_id)))
        self.matcher = llguidance.LLMatcher(self.tokenizer, llguidance.LLMatcher.grammar_from_lark(lark_grammar))

    def allowed_mask(self):
        return self.matcher.compute_logit_bias()

    def accept(self, token_id: int) -> bool:
        return bool(self.matcher.consume_token(int(token_id)))

    def finished(self) -> bool:
        return bool(self.matcher.is_stopped())


class _VocabAdapter:
    def __init__(self, vocab: Sequence[bytes], eos: int):
        self.tokens = list(vocab)
        self.eos_token_id = eos
        self.bos_token_id = None
        self.special_token_ids = [eos]

    def __call__(self, s: str) -> List[int]:
        raise NotImplementedError("canonical tokenisation is not needed for masking")


# ------------------------------------------------------------------------------------------------------------------
# In-tree matcher for the generated tool-call grammar.
#
# The grammar ``tool_call_grammar`` emits is regular once JSON-typed parameter values are taken as "text up to the
# closing tag" (their JSON syntax and schema are checked by the result policy after generation): literals, character
# classes, sequences, alternatives, options and repetition.  That needs no general parser: the tool set is compiled to
# a character NFA (Thompson construction), determinised lazily, and a token is allowed in a state iff feeding its
# characters never leaves the automaton.  Allowed-token masks are computed by walking a character trie of the
# vocabulary (dead prefixes prune whole subtrees) and cached per automaton state, so steady-state cost per generated
# token is one dictionary lookup.  Same contract as the reference's llguidance-backed matcher
# (``hipengine/generation/grammar.py:1-184``): ``allowed_mask`` before sampling, ``accept`` after, ``finished``.

class _NFA:
    def __init__(self) -> None:
        self.eps: List[List[int]] = []
        self.edges: List[List[tuple]] = []      # (predicate kind, payload, target)

    def new(self) -> int:
        self.eps.append([])
        self.edges.append([])
        return len(self.eps) - 1

    # fragments are (start, end) pairs
    def lit(self, s: str):
        a = cur = self.new()
        for ch in s:
            nxt = self.new()
            self.edges[cur].append(("eq", ch, nxt))
            cur = nxt
        return a, cur

    def cls(self, kind: str, payload: str = ""):
        a, b = self.new(), self.new()
        self.edges[a].append((kind, payload, b))
        return a, b

    def seq(self, *frags):
        frags = [f for f in frags if f is not None]
        if not frags:
            a = self.new()
            return a, a
        for (s0, e0), (s1, _e1) in zip(frags, frags[1:]):
            self.eps[e0].append(s1)
        return frags[0][0], frags[-1][1]

    def alt(self, *frags):
        a, b = self.new(), self.new()
        for s, e in frags:
            self.eps[a].append(s)
            self.eps[e].append(b)
        return a, b

    def opt(self, frag):
        a, b = self.new(), self.new()
        self.eps[a] += [frag[0], b]
        self.eps[frag[1]].append(b)
        return a, b

    def star(self, frag):
        a, b = self.new(), self.new()
        self.eps[a] += [frag[0], b]
        self.eps[frag[1]] += [frag[0], b]
        return a, b

    def plus(self, frag_fn):
        first = frag_fn()
        return self.seq(first, self.star(frag_fn()))


def _match(kind: str, payload: str, ch: str) -> bool:
    if kind == "eq":
        return ch == payload
    if kind == "not":
        return ch not in payload
    if kind == "in":
        return ch in payload
    return False


class ToolCallAutomaton:
    """Character automaton of the XML tool-call format for a tool list (see ``tool_call_grammar`` for the format)."""

    def __init__(self, tools: Sequence[Mapping[str, Any]], allow_text_before: bool = True, parallel: bool = True,
                 only: Optional[str] = None):
        n = self.nfa = _NFA()
        ws = lambda: n.star(n.cls("in", " \t\n"))
        digits = lambda: n.plus(lambda: n.cls("in", "0123456789"))

        def integer():
            return n.seq(n.opt(n.lit("-")), n.alt(n.lit("0"), n.seq(n.cls("in", "123456789"),
                                                                   n.star(n.cls("in", "0123456789")))))

        def number():
            frac = n.opt(n.seq(n.lit("."), digits()))
            exp = n.opt(n.seq(n.cls("in", "eE"), n.opt(n.cls("in", "+-")), digits()))
            return n.seq(integer(), frac, exp)

        def value(schema: Mapping[str, Any]):
            t = schema.get("type")
            if "enum" in schema:
                return n.alt(*[n.lit(v if isinstance(v, str) else json.dumps(v)) for v in schema["enum"]])
            if t == "integer":
                return integer()
            if t == "number":
                return number()
            if t == "boolean":
                return n.alt(n.lit("true"), n.lit("false"))
            return n.star(n.cls("not", "<"))         # strings, and JSON-typed values (validated after generation)

        fns = []
        for tool in tools:
            fn = tool.get("function", tool)
            fname = fn.get("name", "")
            if not _NAME_OK.match(fname):
                raise ValueError(f"tool name {fname!r} cannot be expressed in the tool-call grammar")
            if only is not None and fname != only:
                continue
            params = fn.get("parameters") or {}
            required = set(params.get("required") or [])
            parts = []
            for key, sch in (params.get("properties") or {}).items():
                if not _NAME_OK.match(key):
                    raise ValueError(f"parameter name {key!r} cannot be expressed in the tool-call grammar")
                p = n.seq(n.lit("<parameter=" + key + ">"), ws(), value(sch or {}), ws(), n.lit("</parameter>"), ws())
                parts.append(p if key in required else n.opt(p))
            fns.append(n.seq(n.lit("<function=" + fname + ">"), ws(), *parts, n.lit("</function>")))
        if not fns:
            raise ValueError("no tool matches the requested tool choice")
        body = n.alt(*fns)
        first = n.seq(n.lit("<tool_call>"), ws(), body, ws(), n.lit("</tool_call>"))
        if parallel:
            # further calls re-enter the same function alternation through epsilon edges (no copy of the bodies)
            more_open = n.seq(ws(), n.lit("<tool_call>"), ws())
            n.eps[first[1]].append(more_open[0])
            n.eps[more_open[1]].append(body[0])
        start = n.seq(n.opt(n.plus(lambda: n.cls("not", "<"))), first) if allow_text_before else first
        self.start_set = self._closure({start[0]})
        self.accept = start[1]
        self._dfa: Dict[frozenset, Dict[str, Optional[frozenset]]] = {}

    def _closure(self, states) -> frozenset:
        out, stack = set(states), list(states)
        while stack:
            s = stack.pop()
            for t in self.nfa.eps[s]:
                if t not in out:
                    out.add(t)
                    stack.append(t)
        return frozenset(out)

    def step(self, state: frozenset, ch: str) -> Optional[frozenset]:
        row = self._dfa.setdefault(state, {})
        if ch in row:
            return row[ch]
        nxt = set()
        for s in state:
            for kind, payload, t in self.nfa.edges[s]:
                if _match(kind, payload, ch):
                    nxt.add(t)
        res = self._closure(nxt) if nxt else None
        row[ch] = res
        return res

    def accepting(self, state: frozenset) -> bool:
        return self.accept in state


class VocabTrie:
    """Character trie over the decoded strings of a vocabulary (built once per tokenizer)."""

    __slots__ = ("children", "tokens", "size")

    def __init__(self, vocab: Optional[Sequence[str]] = None):
        self.children: Dict[str, "VocabTrie"] = {}
        self.tokens: List[int] = []
        self.size = 0
        if vocab is not None:
            self.size = len(vocab)
            for tid, s in enumerate(vocab):
                if not s:
                    continue                      # tokens that decode to nothing (specials) are never allowed
                node = self
                for ch in s:
                    nxt = node.children.get(ch)
                    if nxt is None:
                        nxt = node.children[ch] = VocabTrie()
                    node = nxt
                node.tokens.append(tid)


class ToolCallMatcher:
    """Token-level constraint for one request: ``allowed_mask()`` before sampling, ``accept(token)`` after.

    ``vocab`` is the decoded string of every token id.  The end-of-sequence token is allowed exactly when the text so
    far is a complete match (free text followed by whole tool calls)."""

    def __init__(self, automaton: ToolCallAutomaton, vocab: Sequence[str], eos_token_id: Optional[int],
                 trie: Optional[VocabTrie] = None):
        self.auto = automaton
        self.vocab = vocab
        self.eos = eos_token_id
        self.trie = trie if trie is not None else VocabTrie(vocab)
        self.state: Optional[frozenset] = automaton.start_set
        self._masks: Dict[frozenset, Any] = automaton.__dict__.setdefault("_mask_cache", {})

    def allowed_mask(self):
        import torch
        st = self.state
        if st is None:
            m = torch.zeros(len(self.vocab), dtype=torch.bool)
            if self.eos is not None:
                m[self.eos] = True
            return m
        m = self._masks.get(st)
        if m is None:
            ok: List[int] = []
            stack = [(self.trie, st)]
            step = self.auto.step
            while stack:
                node, s = stack.pop()
                for ch, child in node.children.items():
                    ns = step(s, ch)
                    if ns is None:
                        continue
                    if child.tokens:
                        ok.extend(child.tokens)
                    if child.children:
                        stack.append((child, ns))
            m = torch.zeros(len(self.vocab), dtype=torch.bool)
            if ok:
                m[torch.tensor(ok, dtype=torch.long)] = True
            if self.eos is not None:
                m[self.eos] = self.auto.accepting(st)
            self._masks[st] = m
        return m

    def accept(self, token_id: int) -> bool:
        """Advance by one generated token; False (and a dead state) if the token is not allowed here."""
        if self.state is None:
            return False
        if self.eos is not None and int(token_id) == self.eos:
            ok = self.auto.accepting(self.state)
            return ok
        s = self.state
        text = self.vocab[int(token_id)]
        if not text:
            self.state = None
            return False
        for ch in text:
            s = self.auto.step(s, ch)
            if s is None:
                self.state = None
                return False
        self.state = s
        return True

    def finished(self) -> bool:
        return self.state is not None and self.auto.accepting(self.state)

    def dead(self) -> bool:
        return self.state is None


_TRIE_CACHE: Dict[int, tuple] = {}


def tool_call_matcher(tools: Sequence[Mapping[str, Any]], tokenizer, eos_token_id: Optional[int],
                      allow_text_before: bool = True, parallel: bool = True,
                      only: Optional[str] = None) -> ToolCallMatcher:
    """Matcher for ``tools`` over ``tokenizer``'s vocabulary (the decoded vocabulary and its trie are cached per
    tokenizer object)."""
    key = id(tokenizer)
    ent = _TRIE_CACHE.get(key)
    if ent is None:
        n = int(getattr(tokenizer, "vocab_size", 0) or len(getattr(tokenizer, "vocab", [])))
        vocab = [tokenizer.decode([i]) for i in range(n)]
        ent = _TRIE_CACHE[key] = (vocab, VocabTrie(vocab))
    vocab, trie = ent
    return ToolCallMatcher(ToolCallAutomaton(tools, allow_text_before, parallel, only), vocab, eos_token_id, trie)
