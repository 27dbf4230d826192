"""Text around the token loop (no GPU): whole-character streaming, the chat turn, the chat loop's commands,
and a session's pieces and turns over a scripted engine with a byte-level stand-in tokenizer."""
import io
from types import SimpleNamespace

import pytest

from nncpu_b200.cli import Options, chat_loop, parse_chat_line, parse_options
from nncpu_b200.errors import ContextFull, InvalidArgument
from nncpu_b200.sampling import GenerateParams, SamplerParams, StopReason
from nncpu_b200.session import Piece, Session, SessionParams
from nncpu_b200.text import TextStream, Tokenizer, chat_turn, end_token_ids, utf8_take

from test_generate_loop import FakeEngine

IM_START, IM_END = 256, 257


class ByteTokenizer(Tokenizer):
    """Token i < 256 is the byte i; 256 and 257 are the ChatML markers."""

    def encode(self, text):
        return list(text.encode("utf-8"))

    def token_bytes(self, token):
        return bytes([token]) if token < 256 else b""

    def special_id(self, name):
        return {"<|im_start|>": IM_START, "<|im_end|>": IM_END}.get(name)


def test_utf8_take_holds_back_a_cut_character():
    p = bytearray("aé".encode()[:2])          # 'a' and the first byte of 'é'
    assert utf8_take(p) == "a" and p == b"\xc3"
    p += b"\xa9"
    assert utf8_take(p) == "é" and p == b""
    # a four-byte character that arrives in three parts comes out once, whole
    s = TextStream()
    b = "🙂".encode()
    assert [s.write(b[:1]), s.write(b[1:3]), s.write(b[3:])] == ["", "", "🙂"]
    # invalid bytes become U+FFFD by maximal subparts; a cut character at the very end too
    assert utf8_take(bytearray(b"\xffa\xe2\x28")) == "�a�("
    assert utf8_take(bytearray(b"ok\xe2\x82"), fin=True) == "ok�"
    assert utf8_take(bytearray(b"\xc0\xaf")) == "��"      # overlong forms are refused
    assert utf8_take(bytearray(b"\xed\xa0\x80")) == "���"  # surrogates too
    s = TextStream()
    assert s.write(b"x\xf0\x9f") == "x" and s.finish() == "�"


def test_chat_turn_tokens():
    t = ByteTokenizer()
    enc = t.encode
    first = chat_turn(t, "hi", first=True, reply_closed=False, system="be brief")
    assert first == ([IM_START] + enc("system\nbe brief") + [IM_END] + enc("\n") + [IM_START] + enc("user\nhi")
                     + [IM_END] + enc("\n") + [IM_START] + enc("assistant\n"))
    again = chat_turn(t, "more", first=False, reply_closed=False)
    assert again[:2] == [IM_END] + enc("\n") and again[2] == IM_START     # the cut-off reply is closed first
    closed = chat_turn(t, "more", first=False, reply_closed=True, reply_open="<think>\n\n</think>\n\n")
    assert closed[0] == enc("\n")[0] and closed[1] == IM_START
    assert closed[-len(enc("assistant\n<think>\n\n</think>\n\n")):] == enc("assistant\n<think>\n\n</think>\n\n")
    assert end_token_ids(t) == [IM_END]
    with pytest.raises(InvalidArgument, match="ChatML"):
        chat_turn(SimpleNamespace(special_id=lambda n: None), "x", True, False)


def test_chat_line_commands():
    assert parse_chat_line("  \n") == ("empty", "")
    assert parse_chat_line("/exit\n") == ("exit", "") and parse_chat_line("/bye") == ("exit", "")
    assert parse_chat_line("/help") == ("help", "") and parse_chat_line("/reset ") == ("reset", "")
    assert parse_chat_line("/nope") == ("unknown", "/nope")
    assert parse_chat_line("/usr/bin is a path") == ("message", "/usr/bin is a path")
    o = parse_options(["chat", "-m", "dir", "-sys", "short answers", "--perf"])
    assert o.mode == "chat" and o.model == "dir" and o.system_prompt == "short answers" and o.perf


class ReplyScript:
    """A chooser that writes the next reply of ``replies`` byte by byte, then <|im_end|>."""
    replies = []

    def __init__(self, params, seed, vocab):
        self.bytes = list(ReplyScript.replies.pop(0)) + [IM_END]

    def choose(self, logits, indices):
        return [self.bytes.pop(0)]


class ScriptedSession(Session):
    _make_sampler = staticmethod(ReplyScript)


class OwnEngine(FakeEngine):
    """The scripted engine with what a session needs besides: a cache that answers length and truncate."""

    def __init__(self, **kw):
        super().__init__(**kw)
        eng = self
        self.cache = SimpleNamespace(length=lambda s: eng.held[s], truncate=lambda s, n: eng.held.__setitem__(s, n))

    def check_status(self):
        pass


def make_session(n_ctx=200, **params):
    model = SimpleNamespace(spec=SimpleNamespace(stop_token_ids=(), vocab_size=258, max_positions=4096))
    engine = OwnEngine(max_seq_len=n_ctx, n_pages=64)
    return ScriptedSession(model, SessionParams(n_ctx=n_ctx, seed=1, max_batch=1, **params), ByteTokenizer(), engine), engine


def test_session_pieces_carry_whole_characters():
    s, engine = make_session()
    ReplyScript.replies = ["zé🙂".encode()]
    pieces = []
    res = s.extend(list(b"hi"), GenerateParams(0, SamplerParams.greedy()), lambda p: pieces.append(p) or True)
    assert res.stop == StopReason.END_OF_TURN and res.n_generated == len("zé🙂".encode())
    assert [p.text for p in pieces] == ["z", "", "é", "", "", "", "🙂"]
    assert all(isinstance(p, Piece) and p.index == 0 for p in pieces)
    # a reply cut in the middle of a character ends with a last piece that has no token
    ReplyScript.replies = ["a🙂".encode()]
    pieces = []
    res = s.extend(list(b"x"), GenerateParams(3, SamplerParams.greedy()), lambda p: pieces.append(p) or True)
    assert res.stop == StopReason.MAX_TOKENS
    assert [(p.token is None, p.text) for p in pieces] == [(False, "a"), (False, ""), (False, ""), (True, "�")]


def test_chat_turns_keep_the_conversation_and_reset_forgets_it():
    s, engine = make_session(system_prompt="sys")
    t = s.tokenizer
    ReplyScript.replies = [b"one", b"two", b"three"]
    text = []
    r1 = s.chat("a", GenerateParams(0, SamplerParams.greedy()), lambda p: text.append(p.text) or True)
    turn1 = chat_turn(t, "a", True, False, "sys")
    assert "".join(text) == "one" and r1.n_prompt == len(turn1)
    assert s.tokens() == turn1 + list(b"one") + [IM_END]
    assert engine.steps[0] == [len(turn1)]                 # the whole first turn in one step
    n_steps = len(engine.steps)
    r2 = s.chat("b", GenerateParams(0, SamplerParams.greedy()))
    turn2 = chat_turn(t, "b", False, True)                 # the model closed its reply itself
    # only what is new is evaluated: the reply's last token (which waited) and the turn
    assert engine.steps[n_steps] == [1 + len(turn2)] and r2.n_prompt == 1 + len(turn2)
    assert s.tokens() == turn1 + list(b"one") + [IM_END] + turn2 + list(b"two") + [IM_END]
    assert len(engine.held) == 1                           # the session's own slot stays
    s.reset()
    assert not engine.held and s.tokens() == []
    r3 = s.chat("c", GenerateParams(2, SamplerParams.greedy()))
    assert r3.stop == StopReason.MAX_TOKENS and s.tokens()[-2:] == list(b"th")
    turn4 = chat_turn(t, "d", False, False)
    assert turn4[0] == IM_END                              # a reply that was cut is closed by the next turn
    with pytest.raises(InvalidArgument, match="tokenizer"):
        Session.chat(SimpleNamespace(tokenizer=None), "x")


def test_context_full_is_refused_before_anything_changes_and_the_chat_loop_starts_afresh():
    s, engine = make_session(n_ctx=60)
    ReplyScript.replies = [b"ok", b"fine", b"again"]
    s.chat("first", GenerateParams(0, SamplerParams.greedy()))
    before = s.tokens()
    with pytest.raises(ContextFull):
        s.chat("x" * 40, GenerateParams(0, SamplerParams.greedy()))
    assert s.tokens() == before
    out, err = io.StringIO(), io.StringIO()
    lines = iter(["/help\n", "x" * 20 + "\n", "/nope\n", "/reset\n", "hello\n", "/exit\n", "never read\n"])
    assert chat_loop(s, Options(), lines, out, err) == 0
    assert out.getvalue() == "fine\nagain\n"
    e = err.getvalue()
    assert "/reset" in e and "starts afresh" in e and "Unknown command /nope" in e and "(new conversation)" in e
    assert e.count("tok/s") == 2                           # a line of figures after each reply
