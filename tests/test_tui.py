"""Deployment form (``ftllm tui``): command-line building, validation, saved configurations, path completion and the
interactive loop driven by a scripted screen."""
import os

from fastllm_b200 import tui
from fastllm_b200.tui import KEY_DOWN, KEY_ENTER, KEY_ESC, KEY_RIGHT, KEY_TAB, KEY_UP, DeployConfig


def test_build_argv_and_validate(tmp_path):
    m = tmp_path / "model"
    m.mkdir()
    c = DeployConfig(name="a", command="server", model=str(m), device="tp", tp="2", dtype="int4g128", port="9000", api_key="k",
                     enable_moe_hybrid=True, moe_device="cpu", moe_device_layers="12", kv_cache_dtype="fp8_e4m3", hide_input=True,
                     extra_args="--dev_mode", env_vars="FB_PDL=1")
    argv = tui.build_argv(c)
    assert argv[:3] == ["ftllm", "server", str(m)]
    for flag, val in (("--tp", "2"), ("--dtype", "int4g128"), ("--port", "9000"), ("--api_key", "k"), ("--moe_device", "cpu"),
                      ("--moe_device_layers", "12"), ("--kv_cache_dtype", "fp8_e4m3"), ("--model_name", "model")):
        assert argv[argv.index(flag) + 1] == val
    assert "--hide_input" in argv and argv[-1] == "--dev_mode" and "--device" not in argv
    assert tui.build_command(c).startswith("FB_PDL=1 ftllm server")
    assert tui.validate(c) == []
    # the built command line is accepted by the real parser
    from fastllm_b200.serving.server import add_server_args
    from fastllm_b200.util import make_normal_parser

    p = make_normal_parser()
    add_server_args(p)
    a = p.parse_args(argv[2:])
    assert a.tp == "2" and a.port == 9000 and a.moe_device == "cpu"
    bad = DeployConfig(command="server", model="/nonexistent/x", port="70000", device="tp", tp="two", gpu_mem_ratio="1.5", top_k="x",
                       env_vars="1A=b")
    errs = " | ".join(tui.validate(bad))
    for frag in ("does not exist", "port", "tensor parallel", "GPU memory ratio", "top_k", "environment"):
        assert frag in errs
    pp = DeployConfig(command="run", model=str(m), device="cudapp", cudapp="2")
    assert "{'cuda:0': 1, 'cuda:1': 1}" in tui.build_argv(pp)


def test_saved_configs_and_completion(tmp_path):
    store = str(tmp_path / "cfg" / "list.json")
    cs = [DeployConfig(name="one", model="/m1"), DeployConfig(name="two", command="run", model="/m2")]
    tui.save_configs(cs, store)
    back = tui.load_configs(store)
    assert [c.name for c in back] == ["one", "two"] and back[1].command == "run"
    assert tui.next_name(back + [DeployConfig(name="config 1")]) == "config 2"
    (tmp_path / "models" / "qwen3").mkdir(parents=True)
    (tmp_path / "models" / "qwen2").mkdir()
    (tmp_path / "models" / "notes.txt").write_text("x")
    base = str(tmp_path / "models") + os.sep
    assert tui.complete_path(base + "qw") == [base + "qwen2" + os.sep, base + "qwen3" + os.sep]
    assert tui.complete_path(base + "n") == [base + "notes.txt"]
    assert tui.complete_path(base + "n", dirs_only=True) == []


class ScriptScreen:
    def __init__(self, keys):
        self.keys = list(keys)
        self.frames = []
        self.cur = []

    def size(self):
        return 50, 160

    def clear(self):
        self.cur = []

    def put(self, y, x, text, bold=False, reverse=False):
        self.cur.append((y, x, text, reverse))

    def refresh(self):
        self.frames.append(list(self.cur))

    def key(self):
        return self.keys.pop(0) if self.keys else KEY_ESC


def test_interactive_flow_creates_edits_and_launches(tmp_path):
    m = tmp_path / "mymodel"
    m.mkdir()
    store = str(tmp_path / "store.json")
    partial = str(tmp_path / "mym")
    keys = ["n",                                             # new configuration -> form
            KEY_DOWN, KEY_RIGHT,                             # command: server -> run
            KEY_DOWN, KEY_ENTER, *partial, KEY_TAB, KEY_ENTER,   # model path with tab completion
            KEY_UP, KEY_UP, KEY_UP, KEY_UP,                  # wrap around to the buttons: ... launch is 3 up from 'name'? go to launch
            ]
    scr = ScriptScreen(keys)
    ui = tui.DeployTUI(scr, configs=[], store_path=store)
    # drive manually: after the scripted keys the selection sits on a button row; press enter until the form returns
    action, cfg = None, None
    scr.keys += [KEY_ENTER]
    action, cfg = ui.run()
    assert cfg is None or cfg.command == "run"
    saved = tui.load_configs(store)
    assert saved and saved[0].command == "run" and saved[0].model == str(m) + os.sep
    # reopen the saved configuration and use the print button
    fields = tui.visible_fields(saved[0], False)
    scr2 = ScriptScreen([KEY_ENTER] + [KEY_DOWN] * (len(fields) + 2) + [KEY_ENTER])
    action, cfg = tui.DeployTUI(scr2, store_path=store).run()
    assert action == "print" and cfg.model == str(m) + os.sep
    assert any("ftllm run" in t for frame in scr2.frames for _, _, t, _ in frame)


def test_plain_screen_reads_line_commands(tmp_path):
    import io

    inp = io.StringIO("n\nd\nr\nq\nq\n")
    out = io.StringIO()
    ui = tui.DeployTUI(tui.PlainScreen(inp, out), configs=[], store_path=str(tmp_path / "s.json"))
    action, _ = ui.run()
    assert action == "quit" and "deployments" in out.getvalue() and ui.configs[0].command == "run"
