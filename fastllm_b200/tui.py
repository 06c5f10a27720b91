"""``ftllm tui`` (also what ``ftllm`` without arguments starts): a terminal form that builds, saves and launches
deployment commands.

The reference's TUI is a deployment configurator, not a chat window (tools/fastllm_pytools/tui.py: ``DeployConfig``
:86-128, ``build_fastllm_argv`` :997-1047, ``validate_config`` :1057+, saved configurations :931-956, path completion
:958-995, the curses front end :1158+).  The same pieces are here:

* ``DeployConfig`` -- one saved deployment (command, model, devices / tensor parallel, dtypes, limits, server options);
* ``build_argv`` / ``build_command`` -- the ``ftllm`` command line it stands for; ``validate`` -- what is wrong with it;
* ``load_configs`` / ``save_configs`` -- the list kept in ``~/.cache/fastllm_b200/tui_configs.json``;
* ``complete_path`` -- tab completion for the model path field;
* ``DeployTUI`` -- the interactive part.  It talks to a small *screen* interface (``size``, ``clear``, ``put``, ``refresh``,
  ``key``), implemented over curses for terminals and over plain stdin/stdout for ``--plain``; tests drive it with a
  scripted screen.
"""
from __future__ import annotations

import dataclasses
import json
import os
import shlex
import sys
from dataclasses import dataclass, field

COMMANDS = ["server", "run", "webui", "bench", "export"]
DEVICES = ["cuda", "cuda:N", "tp", "cudapp", "cpu", "custom"]
DTYPES = ["auto", "float16", "bfloat16", "int8", "int4g128", "fp8", "custom"]
KV_DTYPES = ["auto", "float16", "bfloat16", "fp8_e4m3"]


@dataclass
class DeployConfig:
    name: str = ""
    command: str = "server"
    model: str = ""
    model_name: str = ""
    host: str = "0.0.0.0"
    port: str = "8080"
    device: str = "cuda"
    cuda_device_id: str = "0"
    tp: str = "2"
    cudapp: str = "2"
    device_custom: str = ""
    enable_moe_hybrid: bool = False
    moe_device: str = "cpu"
    moe_device_layers: str = "10000"
    dtype: str = "auto"
    dtype_custom: str = ""
    moe_dtype: str = "auto"
    moe_dtype_custom: str = ""
    gpu_mem_ratio: str = "0.9"
    chunked_prefill_size: str = "auto"
    kv_cache_dtype: str = "auto"
    tokens: str = "auto"
    threads: str = "auto"
    max_batch: str = "auto"
    max_context_length: str = "auto"
    temperature: str = ""
    top_p: str = ""
    top_k: str = ""
    repeat_penalty: str = ""
    api_key: str = ""
    hide_input: bool = False
    cache_dir: str = ""
    ori: str = ""
    output: str = ""
    extra_args: str = ""
    env_vars: str = ""


@dataclass
class Field:
    key: str
    label: str
    kind: str = "text"                 # text | choice | bool | path
    choices: list = field(default_factory=list)
    advanced: bool = False
    visible: object = None             # callable(DeployConfig) -> bool

    def shown(self, cfg: DeployConfig, advanced: bool) -> bool:
        if self.advanced and not advanced:
            return False
        return True if self.visible is None else bool(self.visible(cfg))


FIELDS = [
    Field("name", "Configuration name"),
    Field("command", "Command", "choice", COMMANDS),
    Field("model", "Model path (HF folder / .flm / .gguf)", "path"),
    Field("device", "Main device", "choice", DEVICES),
    Field("cuda_device_id", "GPU id", visible=lambda c: c.device == "cuda:N"),
    Field("tp", "Tensor parallel (count or id list)", visible=lambda c: c.device == "tp"),
    Field("cudapp", "Layer split over N GPUs", visible=lambda c: c.device == "cudapp"),
    Field("device_custom", "Device string", visible=lambda c: c.device == "custom"),
    Field("dtype", "Weight dtype", "choice", DTYPES),
    Field("dtype_custom", "Weight dtype (custom)", visible=lambda c: c.dtype == "custom"),
    Field("enable_moe_hybrid", "Routed experts on the host (hybrid)", "bool"),
    Field("moe_device", "Expert device", "choice", ["cpu", "numa", "disk"], visible=lambda c: c.enable_moe_hybrid),
    Field("moe_device_layers", "Layers with host experts", visible=lambda c: c.enable_moe_hybrid),
    Field("moe_dtype", "Expert dtype", "choice", DTYPES, advanced=True),
    Field("moe_dtype_custom", "Expert dtype (custom)", advanced=True, visible=lambda c: c.moe_dtype == "custom"),
    Field("host", "Host", visible=lambda c: c.command == "server"),
    Field("port", "Port", visible=lambda c: c.command in ("server", "webui")),
    Field("model_name", "Served model name", visible=lambda c: c.command == "server"),
    Field("api_key", "API key", visible=lambda c: c.command == "server"),
    Field("output", "Export output path", "path", visible=lambda c: c.command == "export"),
    Field("gpu_mem_ratio", "GPU memory ratio", advanced=True),
    Field("kv_cache_dtype", "KV cache dtype", "choice", KV_DTYPES, advanced=True),
    Field("chunked_prefill_size", "Chunked prefill size", advanced=True),
    Field("tokens", "KV token capacity", advanced=True),
    Field("max_batch", "Max batch", advanced=True),
    Field("max_context_length", "Max context length", advanced=True, visible=lambda c: c.command == "server"),
    Field("threads", "CPU threads", advanced=True),
    Field("temperature", "Default temperature", advanced=True, visible=lambda c: c.command in ("server", "run")),
    Field("top_p", "Default top_p", advanced=True, visible=lambda c: c.command in ("server", "run")),
    Field("top_k", "Default top_k", advanced=True, visible=lambda c: c.command in ("server", "run")),
    Field("repeat_penalty", "Default repeat penalty", advanced=True, visible=lambda c: c.command in ("server", "run")),
    Field("hide_input", "Hide request text in logs", "bool", advanced=True, visible=lambda c: c.command == "server"),
    Field("cache_dir", "Download cache dir", "path", advanced=True),
    Field("ori", "Original HF folder (for .gguf)", "path", advanced=True, visible=lambda c: c.model.endswith(".gguf")),
    Field("extra_args", "Extra arguments", advanced=True),
    Field("env_vars", "Environment (K=V K2=V2)", advanced=True),
]


def visible_fields(cfg: DeployConfig, advanced: bool) -> list[Field]:
    return [f for f in FIELDS if f.shown(cfg, advanced)]


# ---------------------------------------------------------------------------------------------------------------
# config -> command line
# ---------------------------------------------------------------------------------------------------------------
def _opt(argv, name, value, auto=("", "auto")):
    v = str(value).strip()
    if v not in auto:
        argv += [name, v]


def _custom(value, custom):
    return custom.strip() if value == "custom" else value


def parse_env_vars(text: str) -> dict:
    out = {}
    for part in shlex.split(text or ""):
        if "=" not in part:
            raise ValueError(f"'{part}' is not KEY=VALUE")
        k, v = part.split("=", 1)
        if not k or not (k[0].isalpha() or k[0] == "_") or not all(ch.isalnum() or ch == "_" for ch in k):
            raise ValueError(f"'{k}' is not a valid variable name")
        out[k] = v
    return out


def device_args(cfg: DeployConfig) -> tuple[str, str]:
    """(``--device`` value, ``--tp`` value) of the main-device choice."""
    d = cfg.device
    if d == "cuda:N":
        return f"cuda:{cfg.cuda_device_id.strip() or '0'}", ""
    if d == "tp":
        return "", cfg.tp.strip()
    if d == "cudapp":
        n = int(cfg.cudapp) if cfg.cudapp.strip().isdigit() else 2
        return json.dumps({f"cuda:{i}": 1 for i in range(n)}).replace('"', "'"), ""
    if d == "custom":
        return cfg.device_custom.strip(), ""
    return d, ""


def build_argv(cfg: DeployConfig) -> list[str]:
    argv = ["ftllm", cfg.command]
    model = os.path.expanduser(cfg.model.strip())
    if model:
        argv.append(model)
    device, tp = device_args(cfg)
    _opt(argv, "--device", device, auto=("", "cuda"))
    _opt(argv, "--tp", tp)
    if cfg.enable_moe_hybrid:
        _opt(argv, "--moe_device", cfg.moe_device)
        _opt(argv, "--moe_device_layers", cfg.moe_device_layers)
    _opt(argv, "--dtype", _custom(cfg.dtype, cfg.dtype_custom))
    _opt(argv, "--moe_dtype", _custom(cfg.moe_dtype, cfg.moe_dtype_custom))
    _opt(argv, "--gpu_mem_ratio", cfg.gpu_mem_ratio, auto=("", "auto", "0.9"))
    _opt(argv, "--chunked_prefill_size", cfg.chunked_prefill_size)
    _opt(argv, "--kv_cache_dtype", cfg.kv_cache_dtype)
    _opt(argv, "--tokens", cfg.tokens)
    _opt(argv, "-t", cfg.threads)
    _opt(argv, "--max_batch", cfg.max_batch)
    _opt(argv, "--cache_dir", os.path.expanduser(cfg.cache_dir.strip()))
    if cfg.model.endswith(".gguf"):
        _opt(argv, "--ori", os.path.expanduser(cfg.ori.strip()))
    if cfg.command in ("server", "run"):
        for k in ("temperature", "top_p", "top_k", "repeat_penalty"):
            _opt(argv, "--" + k, getattr(cfg, k))
    if cfg.command == "server":
        _opt(argv, "--model_name", cfg.model_name or os.path.basename(model.rstrip("/")))
        _opt(argv, "--host", cfg.host)
        _opt(argv, "--port", cfg.port)
        _opt(argv, "--api_key", cfg.api_key)
        _opt(argv, "--max_context_length", cfg.max_context_length)
        if cfg.hide_input:
            argv.append("--hide_input")
    elif cfg.command == "webui":
        _opt(argv, "--port", cfg.port)
    elif cfg.command == "export":
        _opt(argv, "-o", os.path.expanduser(cfg.output.strip()))
    if cfg.extra_args.strip():
        argv += shlex.split(cfg.extra_args)
    return argv


def build_command(cfg: DeployConfig) -> str:
    try:
        env = [f"{k}={shlex.quote(v)}" for k, v in parse_env_vars(cfg.env_vars).items()]
    except ValueError as e:
        env = [f"<bad environment: {e}>"]
    return " ".join(env + [shlex.quote(a) for a in build_argv(cfg)])


def _is_pos_int(v):
    return v.strip().isdigit() and int(v) > 0


def validate(cfg: DeployConfig) -> list[str]:
    errs = []
    model = os.path.expanduser(cfg.model.strip())
    if not model:
        errs.append("model path is empty")
    elif not os.path.exists(model) and cfg.command != "export":
        errs.append(f"model path does not exist: {model}")
    if cfg.command not in COMMANDS:
        errs.append(f"unknown command '{cfg.command}'")
    if cfg.command in ("server", "webui") and not (_is_pos_int(cfg.port) and int(cfg.port) < 65536):
        errs.append("port must be 1..65535")
    if cfg.device == "cuda:N" and not cfg.cuda_device_id.strip().isdigit():
        errs.append("GPU id must be a number")
    if cfg.device == "tp":
        t = cfg.tp.strip()
        ok = t == "auto" or _is_pos_int(t) or (t and all(p.strip().isdigit() for p in t.split(",")))
        if not ok:
            errs.append("tensor parallel must be a count, 'auto' or a list of GPU ids like 0,1")
    if cfg.device == "cudapp" and not _is_pos_int(cfg.cudapp):
        errs.append("layer split needs a GPU count")
    if cfg.device == "custom" and not cfg.device_custom.strip():
        errs.append("custom device string is empty")
    for key, label in (("gpu_mem_ratio", "GPU memory ratio"),):
        v = getattr(cfg, key).strip()
        if v not in ("", "auto"):
            try:
                if not 0 < float(v) <= 1:
                    errs.append(f"{label} must be in (0, 1]")
            except ValueError:
                errs.append(f"{label} must be a number")
    for key in ("chunked_prefill_size", "tokens", "threads", "max_batch", "max_context_length", "moe_device_layers"):
        v = getattr(cfg, key).strip()
        if v not in ("", "auto") and not _is_pos_int(v):
            errs.append(f"{key} must be a positive integer or auto")
    for key in ("temperature", "top_p", "repeat_penalty"):
        v = getattr(cfg, key).strip()
        if v:
            try:
                float(v)
            except ValueError:
                errs.append(f"{key} must be a number")
    if cfg.top_k.strip() and not cfg.top_k.strip().lstrip("-").isdigit():
        errs.append("top_k must be an integer")
    if cfg.command == "export" and not cfg.output.strip():
        errs.append("export needs an output path")
    try:
        parse_env_vars(cfg.env_vars)
    except ValueError as e:
        errs.append(f"environment: {e}")
    return errs


# ---------------------------------------------------------------------------------------------------------------
# saved configurations, path completion
# ---------------------------------------------------------------------------------------------------------------
def configs_path() -> str:
    base = os.environ.get("FASTLLM_CACHEDIR") or os.path.join(os.path.expanduser("~"), ".cache", "fastllm_b200")
    return os.path.join(base, "tui_configs.json")


def load_configs(path: str | None = None) -> list[DeployConfig]:
    path = path or configs_path()
    try:
        data = json.load(open(path, encoding="utf-8"))
    except (OSError, ValueError):
        return []
    names = {f.name for f in dataclasses.fields(DeployConfig)}
    return [DeployConfig(**{k: v for k, v in d.items() if k in names}) for d in data if isinstance(d, dict)]


def save_configs(configs, path: str | None = None) -> None:
    path = path or configs_path()
    os.makedirs(os.path.dirname(path), exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump([dataclasses.asdict(c) for c in configs], f, indent=1, ensure_ascii=False)
    os.replace(tmp, path)


def next_name(configs) -> str:
    used = {c.name for c in configs}
    i = 1
    while f"config {i}" in used:
        i += 1
    return f"config {i}"


def complete_path(prefix: str, dirs_only: bool = False) -> list[str]:
    """Completions of a partly typed path (``~`` expanded for the lookup, kept as typed in the result)."""
    raw = prefix or ""
    exp = os.path.expanduser(raw)
    d, base = (exp, "") if exp.endswith(os.sep) or exp == "" else os.path.split(exp)
    try:
        names = sorted(os.listdir(d or "."))
    except OSError:
        return []
    out = []
    raw_dir = raw[:len(raw) - len(base)] if base else raw
    for n in names:
        if not n.startswith(base) or (n.startswith(".") and not base.startswith(".")):
            continue
        full = os.path.join(d or ".", n)
        isdir = os.path.isdir(full)
        if dirs_only and not isdir:
            continue
        out.append(raw_dir + n + (os.sep if isdir else ""))
    return out


# ---------------------------------------------------------------------------------------------------------------
# screens
# ---------------------------------------------------------------------------------------------------------------
KEY_UP, KEY_DOWN, KEY_LEFT, KEY_RIGHT, KEY_ENTER, KEY_ESC, KEY_TAB, KEY_BACKSPACE = "UP", "DOWN", "LEFT", "RIGHT", "ENTER", "ESC", "TAB", "BS"


class CursesScreen:
    def __init__(self, stdscr):
        import curses

        self.c, self.s = curses, stdscr
        curses.curs_set(0)
        stdscr.keypad(True)
        self.map = {curses.KEY_UP: KEY_UP, curses.KEY_DOWN: KEY_DOWN, curses.KEY_LEFT: KEY_LEFT, curses.KEY_RIGHT: KEY_RIGHT,
                    10: KEY_ENTER, 13: KEY_ENTER, curses.KEY_ENTER: KEY_ENTER, 27: KEY_ESC, 9: KEY_TAB,
                    curses.KEY_BACKSPACE: KEY_BACKSPACE, 127: KEY_BACKSPACE, 8: KEY_BACKSPACE}

    def size(self):
        h, w = self.s.getmaxyx()
        return h, w

    def clear(self):
        self.s.erase()

    def put(self, y, x, text, bold=False, reverse=False):
        h, w = self.size()
        if 0 <= y < h and x < w:
            attr = (self.c.A_BOLD if bold else 0) | (self.c.A_REVERSE if reverse else 0)
            try:
                self.s.addnstr(y, x, text, max(0, w - x - 1), attr)
            except self.c.error:
                pass

    def refresh(self):
        self.s.refresh()

    def key(self):
        k = self.s.get_wch()
        if isinstance(k, str):
            return self.map.get(ord(k), k) if len(k) == 1 else k
        return self.map.get(k, "")


class PlainScreen:
    """Line-oriented fallback (``ftllm tui --plain``, or no terminal): the form is printed, one command per line is read
    (``u`` / ``d`` move, text after ``=`` edits, ``enter`` activates, ``q`` leaves)."""

    def __init__(self, inp=None, out=None):
        self.inp, self.out = inp or sys.stdin, out or sys.stdout
        self.lines = {}
        self.pending = []

    def size(self):
        return 40, 120

    def clear(self):
        self.lines = {}

    def put(self, y, x, text, bold=False, reverse=False):
        self.lines[y] = (">" if reverse else " ") + " " * x + text

    def refresh(self):
        self.out.write("\n".join(self.lines[k] for k in sorted(self.lines)) + "\n")
        self.out.flush()

    def key(self):
        if self.pending:
            return self.pending.pop(0)
        line = self.inp.readline()
        if not line:
            return KEY_ESC
        line = line.rstrip("\n")
        table = {"u": KEY_UP, "d": KEY_DOWN, "l": KEY_LEFT, "r": KEY_RIGHT, "": KEY_ENTER, "enter": KEY_ENTER, "q": KEY_ESC, "tab": KEY_TAB}
        if line in table:
            return table[line]
        if line.startswith("="):
            self.pending = [KEY_ENTER] + list(line[1:]) + [KEY_ENTER]
            return self.pending.pop(0)
        return line[:1]


class DeployTUI:
    """Home screen: saved configurations + [new]; a configuration opens the form; the form's buttons launch, save or delete."""

    def __init__(self, screen, configs=None, store_path: str | None = None):
        self.scr = screen
        self.path = store_path
        self.configs = list(configs) if configs is not None else load_configs(store_path)
        self.advanced = False
        self.message = ""

    # -- drawing ----------------------------------------------------------------------------------------------
    def _draw_home(self, sel):
        s = self.scr
        s.clear()
        s.put(0, 0, "fastllm_b200 -- deployments   (enter: open, n: new, x: delete, q: quit)", bold=True)
        rows = [f"{c.name or '(unnamed)'}   [{c.command}] {c.model}" for c in self.configs] + ["+ new configuration"]
        for i, r in enumerate(rows):
            s.put(2 + i, 2, r, reverse=(i == sel))
        if self.message:
            s.put(4 + len(rows), 0, self.message)
        s.refresh()

    def _draw_form(self, cfg, fields, sel, editing, buf):
        s = self.scr
        s.clear()
        s.put(0, 0, f"{cfg.name or '(unnamed)'}   (enter: edit / activate, left/right: choice, a: advanced, tab: complete path, esc: back)", bold=True)
        y = 2
        for i, f in enumerate(fields):
            v = getattr(cfg, f.key)
            shown = ("[x]" if v else "[ ]") if f.kind == "bool" else (f"< {v} >" if f.kind == "choice" else str(v))
            if editing and i == sel:
                shown = buf + "_"
            s.put(y, 2, f"{f.label:38s} {shown}", reverse=(i == sel))
            y += 1
        buttons = ["[ launch ]", "[ save ]", "[ print command ]"]
        for j, b in enumerate(buttons):
            s.put(y + 1, 2 + 20 * j, b, reverse=(sel == len(fields) + j))
        s.put(y + 3, 0, "$ " + build_command(cfg))
        errs = validate(cfg)
        for k, e in enumerate(errs[:4]):
            s.put(y + 5 + k, 0, "! " + e)
        if self.message:
            s.put(y + 10, 0, self.message)
        s.refresh()

    # -- loops ------------------------------------------------------------------------------------------------
    def run(self):
        """Returns ``("launch", config)``, ``("print", config)`` or ``("quit", None)``."""
        sel = 0
        while True:
            n = len(self.configs) + 1
            sel = max(0, min(sel, n - 1))
            self._draw_home(sel)
            k = self.scr.key()
            if k in (KEY_ESC, "q"):
                return "quit", None
            if k == KEY_UP:
                sel = (sel - 1) % n
            elif k == KEY_DOWN:
                sel = (sel + 1) % n
            elif k == "x" and sel < len(self.configs):
                self.message = f"deleted '{self.configs[sel].name}'"
                del self.configs[sel]
                save_configs(self.configs, self.path)
            elif k == "n" or (k == KEY_ENTER and sel == len(self.configs)):
                cfg = DeployConfig(name=next_name(self.configs))
                self.configs.append(cfg)
                r = self._form(cfg)
                if r is not None:
                    return r
            elif k == KEY_ENTER:
                r = self._form(self.configs[sel])
                if r is not None:
                    return r

    def _form(self, cfg):
        sel, editing, buf = 0, False, ""
        self.message = ""
        while True:
            fields = visible_fields(cfg, self.advanced)
            total = len(fields) + 3
            sel = max(0, min(sel, total - 1))
            self._draw_form(cfg, fields, sel, editing, buf)
            k = self.scr.key()
            if editing:
                f = fields[sel]
                if k == KEY_ENTER:
                    setattr(cfg, f.key, buf)
                    editing = False
                elif k == KEY_ESC:
                    editing = False
                elif k == KEY_BACKSPACE:
                    buf = buf[:-1]
                elif k == KEY_TAB and f.kind == "path":
                    c = complete_path(buf)
                    if len(c) == 1:
                        buf = c[0]
                    elif c:
                        buf = os.path.commonprefix(c)
                        self.message = "  ".join(os.path.basename(x.rstrip(os.sep)) for x in c[:8])
                elif isinstance(k, str) and len(k) == 1 and k.isprintable():
                    buf += k
                continue
            if k == KEY_ESC:
                save_configs(self.configs, self.path)
                return None
            if k == KEY_UP:
                sel = (sel - 1) % total
            elif k == KEY_DOWN:
                sel = (sel + 1) % total
            elif k == "a":
                self.advanced = not self.advanced
            elif sel < len(fields):
                f = fields[sel]
                if f.kind == "bool" and k in (KEY_ENTER, " ", KEY_LEFT, KEY_RIGHT):
                    setattr(cfg, f.key, not getattr(cfg, f.key))
                elif f.kind == "choice" and k in (KEY_LEFT, KEY_RIGHT, KEY_ENTER):
                    i = f.choices.index(getattr(cfg, f.key)) if getattr(cfg, f.key) in f.choices else 0
                    setattr(cfg, f.key, f.choices[(i + (-1 if k == KEY_LEFT else 1)) % len(f.choices)])
                elif k == KEY_ENTER:
                    editing, buf = True, str(getattr(cfg, f.key))
            elif k == KEY_ENTER:
                which = sel - len(fields)
                save_configs(self.configs, self.path)
                if which == 1:
                    self.message = "saved"
                    continue
                errs = validate(cfg)
                if errs and which == 0:
                    self.message = "fix the problems listed above first"
                    continue
                return ("launch" if which == 0 else "print"), cfg


def launch(cfg: DeployConfig) -> int:
    """Run the configured command in this interpreter (same as typing the printed command line)."""
    from . import cli

    os.environ.update(parse_env_vars(cfg.env_vars))
    return cli.main(build_argv(cfg)[1:]) or 0


def main(plain: bool = False, store_path: str | None = None) -> int:
    if plain or not (sys.stdin.isatty() and sys.stdout.isatty()):
        action, cfg = DeployTUI(PlainScreen(), store_path=store_path).run()
    else:
        import curses

        action, cfg = curses.wrapper(lambda stdscr: DeployTUI(CursesScreen(stdscr), store_path=store_path).run())
    if action == "print":
        print(build_command(cfg))
        return 0
    if action == "launch":
        print("$ " + build_command(cfg), flush=True)
        return launch(cfg)
    return 0
