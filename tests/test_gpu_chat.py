"""Chat on the device: turns on the session's own sequence keep their cache, the reply is the plain model's
greedy continuation of the whole conversation, text comes in whole characters, and the command line's chat
loop runs two turns and a /reset through a pipe."""
import subprocess
import sys

import pytest

from conftest import ROOT
from nncpu_b200 import GenerateParams, Model, SamplerParams, Session, SessionParams
from nncpu_b200.text import _byte_level_table, chat_turn, load_tokenizer
from plain_qwen3 import PlainQwen3, argmax_first
from tiny import make_folder

pytestmark = pytest.mark.gpu
tokenizers = pytest.importorskip("tokenizers")


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    """Tiny model B (384 tokens) with a byte-level tokenizer.json: token b < 256 is the byte b, then the two
    ChatML markers; end-of-sequence is <|im_end|> (257)."""
    path = make_folder(tmp_path_factory.mktemp("chat") / "B", "B", seed=21, eos_token_id=257)
    spelled = {b: ch for ch, b in _byte_level_table().items()}
    tok = tokenizers.Tokenizer(tokenizers.models.BPE(vocab={spelled[b]: b for b in range(256)}, merges=[]))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    tok.add_special_tokens(["<|im_start|>", "<|im_end|>"])
    tok.save(str(path / "tokenizer.json"))
    return path


def test_tokenizer_file_round_trip(folder):
    t = load_tokenizer(folder)
    assert t.special_id("<|im_start|>") == 256 and t.special_id("<|im_end|>") == 257 and t.special_id("<x>") is None
    ids = t.encode("hé 🙂\n")
    assert ids == list("hé 🙂\n".encode()) and t.decode(ids) == "hé 🙂\n"
    assert t.token_bytes(0xF0) == b"\xf0" and t.token_bytes(257) == b""


def test_turns_continue_the_conversation_from_its_cache(folder):
    plain = PlainQwen3(folder)
    tok = load_tokenizer(folder)
    session = Session(Model.load(folder, dtype="float32"), SessionParams(n_ctx=256, seed=1, max_batch=1,
                                                                         system_prompt="s"), tokenizer=tok)
    greedy = GenerateParams(10, SamplerParams.greedy())
    context = []
    for n, message in enumerate(["hi", "and then?", "ok"]):
        closed = bool(context) and context[-1] == 257
        context += chat_turn(tok, message, n == 0, closed, "s")
        held = session.n_past()
        text = []
        res = session.chat(message, greedy, lambda p: text.append(p.text) or True)
        assert res.n_prompt == len(context) - held              # only what is new was evaluated
        want, seq = [], list(context)
        for _ in range(10):
            t = argmax_first(plain.logits(seq)[-1])
            seq.append(t)
            if t == 257:
                break
            want.append(t)
        assert res.tokens == want
        context = seq
        assert session.tokens() == context
        assert "".join(text) == tok.decode(want)                # whole characters, nothing lost, nothing twice
    session.reset()
    assert session.n_past() == 0 and session.engine.cache.slots.n_held == 0


def test_chat_loop_through_a_pipe(folder):
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "nncpu-b200"), "chat", "-m", str(folder), "--fp32", "-n", "8",
                        "--temp", "0", "-v"], input="hello\nmore\n/reset\nhello\n/exit\nunread\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    replies = p.stdout.split("\n")[:-1]
    assert len(replies) == 3 and replies[0] == replies[2]       # after /reset the same message gets the same reply
    stats = [ln for ln in p.stderr.splitlines() if "tok/s" in ln]
    assert len(stats) == 3 and "(new conversation)" in p.stderr
    prompts = [int(ln.split("prompt ")[1].split()[0]) for ln in stats]
    assert prompts[0] == prompts[2] and prompts[1] != prompts[0]
