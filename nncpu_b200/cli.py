"""Command line in the manner of ``nncpu``: the reference's option names and
meanings where it has them (crates/nncpu-cli/src/cli.rs:78-131,291-362), and
its token-level harness (crates/nncpu-cli/src/devtools.rs:70-90,632-705) as
``--gen``.

    nncpu-b200 -m DIR --tokens "1 2 3" -n 32            generate from token ids
    nncpu-b200 -m DIR -p TEXT                           answer one message (needs tokenizer.json), streamed
    nncpu-b200 chat -m DIR                              chat: a message per line, /reset /exit /help
    nncpu-b200 --gen DIR "ID ID ..." [N] [CTX]          greedy token-level run with timings
    nncpu-b200 --info DIR                               what the folder holds
    nncpu-b200 --random-weights CONFIG.json SEED OUT    write a model folder with random weights
"""
from __future__ import annotations

import json
import os
import signal
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional

from . import __version__
from .errors import InvalidArgument, NncpuError
from .sampling import GenerateParams, SamplerParams

# flag, fewest and most positional arguments (crates/nncpu-cli/src/cli.rs:78-95)
MODES = {"--help": (0, 0), "-h": (0, 0), "--version": (0, 0), "--gen": (2, 4), "--info": (1, 1),
         "--random-weights": (3, 3)}

VALUE_OPTIONS = {
    "-m": "model", "--model": "model",
    "-p": "prompt", "--prompt": "prompt",
    "-sys": "system_prompt", "--system": "system_prompt",
    "--tokens": "tokens",
    "-n": "n_predict", "--n_predict": "n_predict", "--n-predict": "n_predict",
    "-c": "n_ctx", "--ctx-size": "n_ctx", "--ctx_size": "n_ctx",
    "--temp": "temperature",
    "--top_k": "top_k", "--top-k": "top_k",
    "--top_p": "top_p", "--top-p": "top_p",
    "--min_p": "min_p", "--min-p": "min_p",
    "-s": "seed", "--seed": "seed",
    "-b": "batch", "--batch": "batch", "--batch_size": "batch",
    "--dtype": "dtype",
}
FLAGS = {"--bf16": ("dtype", "bfloat16"), "--fp32": ("dtype", "float32"), "--kv-f32": ("kv_f32", True),
         "--perf": ("perf", True), "-v": ("verbose", True), "--verbose": ("verbose", True)}


@dataclass
class Options:
    mode: str = "generate"
    args: List[str] = field(default_factory=list)
    model: str = ""
    prompt: str = ""
    system_prompt: str = ""     # -sys: instructions for the model, given before the first message
    tokens: str = ""
    n_predict: int = 0          # -n: most tokens per reply; 0 = until a stop token or a full context
    n_ctx: int = 0              # -c: 0 = min(4096, the model's position range)
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    seed: int = 0               # -s: 0 = random
    batch: int = 1              # -b: copies of the prompt generated together
    dtype: str = "bfloat16"
    kv_f32: bool = False
    perf: bool = False
    verbose: bool = False

    def sampler(self) -> SamplerParams:
        return SamplerParams(self.temperature, self.top_k, self.top_p, self.min_p)


def _number(flag: str, text: str, kind):
    try:
        v = kind(text)
    except ValueError:
        raise InvalidArgument(f"{flag}: {text!r} is not a number") from None
    return v


def parse_options(argv: List[str]) -> Options:
    o = Options()
    i = 0
    while i < len(argv):
        a = argv[i]
        if a == "chat" and i == 0:
            o.mode = "chat"
        elif a in MODES:
            lo, hi = MODES[a]
            o.mode = {"-h": "--help"}.get(a, a).lstrip("-")
            rest = []
            while i + 1 < len(argv) and len(rest) < hi and not (argv[i + 1] in VALUE_OPTIONS or argv[i + 1] in FLAGS):
                i += 1
                rest.append(argv[i])
            if len(rest) < lo:
                raise InvalidArgument(f"{a} takes {lo} to {hi} arguments, {len(rest)} given")
            o.args = rest
        elif a in VALUE_OPTIONS:
            if i + 1 >= len(argv):
                raise InvalidArgument(f"{a} needs a value")
            i += 1
            name, text = VALUE_OPTIONS[a], argv[i]
            if name in ("n_predict", "n_ctx", "top_k", "seed", "batch"):
                v = _number(a, text, int)
                if v < 0 and name != "seed":
                    raise InvalidArgument(f"{a}: {v} is negative")
                if name == "seed":
                    v = max(v, 0)  # a seed of 0 or below means random (crates/nncpu-cli/src/cli.rs:229-235)
                if name == "batch" and v < 1:
                    raise InvalidArgument(f"{a}: at least 1")
                setattr(o, name, v)
            elif name in ("temperature", "top_p", "min_p"):
                setattr(o, name, _number(a, text, float))
            elif name == "dtype":
                if text not in ("bfloat16", "bf16", "float32", "fp32"):
                    raise InvalidArgument(f"--dtype: {text!r} is not bfloat16 or float32")
                o.dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(text, text)
            else:
                setattr(o, name, text)
        elif a in FLAGS:
            name, v = FLAGS[a]
            setattr(o, name, v)
        else:
            raise InvalidArgument(f"unknown option {a!r} (see --help)")
        i += 1
    o.sampler().check("options")
    return o


def usage(argv0: str = "nncpu-b200") -> str:
    return f"""nncpu-b200 {__version__} - run Qwen3 models on one B200

usage: {argv0} -m DIR --tokens "ID ID ..."   continue the token ids and exit
       {argv0} -m DIR -p TEXT                answer one message and exit (needs tokenizer.json in DIR)
       {argv0} chat -m DIR                   chat: type a message per line (needs tokenizer.json in DIR)

model:
  -m, --model DIR          a folder with config.json and model.safetensors (or its index and files)
  --bf16                   run in bfloat16 (default)
  --fp32                   run everything in true 32-bit (slow; shows what bfloat16 hides)
  --dtype NAME             bfloat16 or float32
  -c, --ctx-size N         context window in tokens (default: up to 4096)
  --kv-f32                 keep the K/V cache in F32 (default: the run's element type)

generation:
  -p, --prompt TEXT        answer TEXT and exit; the reply goes to stdout as it is written
  -sys, --system TEXT      instructions for the model, given before the first message
  --tokens "ID ID ..."     continue these token ids; the new ids go to stdout
  -n, --n_predict N        most tokens per reply (default: until the reply ends)
  -b, --batch N            generate N copies of the prompt together (default 1)
  --temp X                 sampling temperature; 0 = always the likeliest token (default 0.7)
  --top-k N                sample from the N likeliest tokens; 0 = all (default 40)
  --top-p X                ...that make up probability X (default 0.95)
  --min-p X                ...each at least X times the likeliest (default 0.05)
  -s, --seed N             random seed, for repeatable replies (default: random)
  --perf                   print a table of the time per phase after the reply
  -v, --verbose            show what the library is doing

modes (each runs instead of generation):
  --gen DIR "ID ID ..." [N] [CTX]
                           greedy token-level run: prints every token and the prefill and decode speeds
  --info DIR               the model folder's configuration, sizes and parameter count
  --random-weights CONFIG.json SEED OUT
                           write OUT/config.json and OUT/model.safetensors with random weights
  --version                print the version
"""


def _token_list(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise InvalidArgument(f"token ids must be integers: {text!r}") from None


def _peaks() -> Optional[dict]:
    """The device's measured peaks for the profiler's last column: the JSON file that $NNCPU_B200_PEAKS names,
    or MEASURED_PEAKS.json in the working directory ({"hbm_gbs": ..., "bf16_tflops": ...})."""
    for cand in (os.environ.get("NNCPU_B200_PEAKS"), "MEASURED_PEAKS.json"):
        if cand and Path(cand).exists():
            try:
                d = json.loads(Path(cand).read_text())
                return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}
            except (ValueError, KeyError, TypeError):
                return None
    return None


def _perf_begin(o: Options) -> None:
    if o.perf:
        from . import perf_enable, perf_reset
        perf_enable(True)
        perf_reset()


def _perf_end(o: Options, title: str, n_tokens: int, err) -> None:
    """The phase table after a reply (crates/nncpu-cli/src/chat.rs:232-235)."""
    if o.perf:
        from . import perf_report, perf_reset
        err.write(perf_report(title, n_tokens, _peaks()))
        perf_reset()


def _stats_line(res, verbose: bool, n_predict: int) -> str:
    """The line after a reply: tokens, speed, and why it stopped if that was not the model's own choice
    (crates/nncpu-cli/src/chat.rs:170-231)."""
    from .sampling import StopReason
    note = {StopReason.MAX_TOKENS: f", cut at -n {n_predict}", StopReason.CANCELLED: ", stopped",
            StopReason.CONTEXT_FULL: ", context full: the next message starts afresh"}.get(res.stop, "")
    tps = res.n_generated / res.decode if res.decode > 0 else 0.0
    if verbose:
        return f"[{res.n_generated} tokens, {tps:.1f} tok/s; prompt {res.n_prompt} tokens in {res.prefill:.2f} s{note}]"
    return f"[{res.n_generated} tokens, {tps:.1f} tok/s{note}]"


def run_generate(o: Options, out=sys.stdout, err=sys.stderr) -> int:
    from . import Model, Session, SessionParams
    from .text import load_tokenizer
    if not o.model:
        raise InvalidArgument("no model: pass -m DIR")
    if bool(o.prompt) == bool(o.tokens):
        raise InvalidArgument("pass exactly one of -p TEXT and --tokens \"ID ID ...\"")
    tok = load_tokenizer(o.model) if o.prompt else None
    t0 = time.perf_counter()
    model = Model.load(o.model, dtype=o.dtype)
    if o.verbose:
        print(f"loaded {model.info()} in {time.perf_counter() - t0:.2f} s", file=err)
    session = Session(model, SessionParams(n_ctx=o.n_ctx, seed=o.seed, kv_f32=o.kv_f32, max_batch=o.batch,
                                           system_prompt=o.system_prompt), tokenizer=tok)
    _perf_begin(o)
    params = GenerateParams(o.n_predict, o.sampler())
    if tok is not None:
        # one chat turn on the session's own sequence, streamed in whole characters
        def on_text(p):
            out.write(p.text)
            out.flush()
            return True
        r = session.chat(o.prompt, params, on_text)
        res = [r]
    else:
        def on_piece(p):
            if p.index == 0:
                out.write(f"{p.token} ")
                out.flush()
            return True
        res = session.generate([_token_list(o.tokens)] * o.batch, params, on_piece)
    out.write("\n")
    out.flush()
    if o.perf or o.verbose:
        r = res[0]
        n = sum(x.n_generated for x in res)
        print(f"{r.n_prompt} prompt tokens in {r.prefill:.3f} s ({len(res) * r.n_prompt / max(r.prefill, 1e-9):.1f} tok/s), "
              f"{n} tokens in {r.decode:.3f} s ({n / max(r.decode, 1e-9):.1f} tok/s), stop: {r.stop.value}", file=err)
    _perf_end(o, "reply", sum(x.n_prompt + x.n_generated for x in res), err)
    return 0


CHAT_HELP = """Commands:
  /reset            forget the conversation and start a new one
  /exit             quit (so does the end of the input)
  /help             this list
Ctrl-C stops a reply that is being written.
"""


def parse_chat_line(line: str):
    """What a line typed at the prompt asks for: (kind, text) with kind one of empty, exit, help, reset,
    unknown, message (crates/nncpu-cli/src/chat.rs:253-293)."""
    msg = line.strip(" \t\r\n")
    if msg == "":
        return "empty", ""
    if msg in ("/exit", "/quit", "/bye"):
        return "exit", ""
    if msg in ("/help", "/?"):
        return "help", ""
    if msg in ("/reset", "/clear"):
        return "reset", ""
    if msg.startswith("/") and " " not in msg:
        return "unknown", msg
    return "message", msg


def chat_loop(session, o: Options, lines, out=sys.stdout, err=sys.stderr, interactive: bool = False) -> int:
    """The chat loop over ``lines`` (an iterable of input lines): commands, one turn per message on the
    session's own sequence, whose cache stays between turns, a line of figures after every reply, Ctrl-C wired to
    the session's cancel handle while a reply is written.  A conversation that has filled the context starts
    afresh and the message is tried again (crates/nncpu-cli/src/chat.rs:138-166,302-484)."""
    from .errors import ContextFull
    params = GenerateParams(o.n_predict, o.sampler())
    cancel = session.cancel_handle()

    def turn(message):
        def on_text(p):
            out.write(p.text)
            out.flush()
            return True
        old = None
        try:
            old = signal.signal(signal.SIGINT, lambda *_: cancel.cancel())
        except ValueError:
            pass                     # not the main thread: no Ctrl-C wiring
        try:
            try:
                return session.chat(message, params, on_text)
            except ContextFull:
                if session.n_past() == 0 and not session.tokens():
                    raise
                print(f"(the conversation filled the {session.n_ctx}-token context, so it starts afresh)", file=err)
                session.reset()
                return session.chat(message, params, on_text)
        finally:
            if old is not None:
                signal.signal(signal.SIGINT, old)

    print("Type a message and press Enter. /help lists commands; Ctrl-C stops a reply.", file=err)
    while True:
        if interactive:
            err.write("\n> ")
            err.flush()
        try:
            line = next(lines)
        except StopIteration:
            break
        kind, text = parse_chat_line(line)
        if kind == "exit":
            break
        if kind == "help":
            err.write(CHAT_HELP)
        elif kind == "reset":
            session.reset()
            print("(new conversation)", file=err)
        elif kind == "unknown":
            print(f"Unknown command {text}; /help lists the commands.", file=err)
        elif kind == "message":
            try:
                res = turn(text)
            except NncpuError as e:
                out.write("\n")
                print(f"error ({e.kind}): {e}", file=err)
                continue
            out.write("\n")
            out.flush()
            print(_stats_line(res, o.verbose, o.n_predict), file=err)
            _perf_end(o, "reply", res.n_prompt + res.n_generated, err)
    return 0


def run_chat(o: Options, stdin=None, out=sys.stdout, err=sys.stderr) -> int:
    from . import Model, Session, SessionParams
    from .text import load_tokenizer
    if not o.model:
        raise InvalidArgument("no model: pass -m DIR")
    tok = load_tokenizer(o.model)
    model = Model.load(o.model, dtype=o.dtype)
    session = Session(model, SessionParams(n_ctx=o.n_ctx, seed=o.seed, kv_f32=o.kv_f32, max_batch=1,
                                           system_prompt=o.system_prompt), tokenizer=tok)
    info = model.info()
    print(f"{o.model} ({info['architecture']}, {info['layers']} layers, {info['dtype']}) - "
          f"{session.n_ctx}-token context", file=err)
    _perf_begin(o)
    stdin = stdin if stdin is not None else sys.stdin
    return chat_loop(session, o, iter(stdin.readline, ""), out, err, interactive=stdin.isatty())


def run_gen(o: Options, out=sys.stdout) -> int:
    """Greedy token-level harness (crates/nncpu-cli/src/devtools.rs:635-705)."""
    from . import Model, Session, SessionParams
    folder, ids = o.args[0], _token_list(o.args[1])
    n = int(o.args[2]) if len(o.args) > 2 else 32
    ctx = int(o.args[3]) if len(o.args) > 3 else max(256, len(ids) + n + 1)
    model = Model.load(folder, dtype=o.dtype)
    session = Session(model, SessionParams(n_ctx=ctx, seed=1, kv_f32=o.kv_f32, max_batch=1))
    _perf_begin(o)
    res = session.generate([ids], GenerateParams(n, SamplerParams.greedy()))[0]
    out.write(" ".join(str(t) for t in res.tokens) + "\n")
    out.write(f"prefill: {res.n_prompt} tokens, {res.prefill * 1e3:.1f} ms ({res.n_prompt / max(res.prefill, 1e-9):.1f} tok/s)\n")
    out.write(f"decode: {res.n_generated} tokens, {res.decode * 1e3:.1f} ms ({res.n_generated / max(res.decode, 1e-9):.1f} tok/s)\n")
    out.write(f"stop: {res.stop.value}\n")
    _perf_end(o, "gen", res.n_prompt + res.n_generated, out)
    return 0


def run_info(o: Options, out=sys.stdout) -> int:
    from .config import load_config
    from .engine.model import parameter_list
    from .weights import check_tensors, open_checkpoint
    cfg = load_config(o.args[0])
    params = parameter_list(cfg.model_spec())
    files, where, label = open_checkpoint(o.args[0])
    try:
        check_tensors({n: files[name].shape(n) for n, name in where.items()}, params, label)
    finally:
        for f in files.values():
            f.close()
    n = 0
    for p in params:
        if p.name in where:
            c = 1
            for s in p.shape:
                c *= s
            n += c
    out.write(json.dumps({"config": cfg.to_dict(), "tensors": len(where), "parameters": n}, indent=2) + "\n")
    return 0


def run_random_weights(o: Options, out=sys.stdout) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_model_folder
    cfg = config_from_dict(json.loads(Path(o.args[0]).read_text()))
    store = torch.float32 if o.dtype == "float32" else torch.bfloat16
    folder = write_model_folder(o.args[2], cfg, int(o.args[1]), store)
    out.write(f"{folder}\n")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        o = parse_options(argv)
        if o.mode == "help" or not argv:
            print(usage())
            return 0
        if o.mode == "version":
            print(__version__)
            return 0
        if o.mode == "gen":
            return run_gen(o)
        if o.mode == "chat":
            return run_chat(o)
        if o.mode == "info":
            return run_info(o)
        if o.mode == "random-weights":
            return run_random_weights(o)
        return run_generate(o)
    except NncpuError as e:
        print(f"error ({e.kind}): {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
