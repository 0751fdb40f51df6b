"""The command line with a stand-in model (no GPU), as the reference tests its CLI with a
fake engine (cmd/tgo/*_test.go; `openEngine` is a variable there, `opener` here)."""
import io

import pytest

from tgo_b200 import cli
from tgo_b200.sampling.policy import DrawStream, Policy


class FakeSession:
    def __init__(self, context, **kw):
        self.context = context
        self.kw = kw
        self.calls = []

    def complete(self, prompt, policy):
        self.calls.append((list(prompt), policy))
        for i in range(policy.max_tokens):
            yield 100 + i


class FakeModel:
    class spec:
        vocab_size = 1000
    info = {"architecture": "Qwen3ForCausalLM", "weight_bytes": 10 ** 9}

    stop_ids = [7, 9]

    def __init__(self):
        self.sessions = []
        self.generated = []

    def new_session(self, context=4096, **kw):
        self.sessions.append(FakeSession(context, **kw))
        return self.sessions[-1]

    def generate(self, prompts, policies, **kw):
        self.generated.append((prompts, policies, kw))
        return [[200 + i] * policies[i].max_tokens for i in range(len(prompts))]


def run(argv):
    out, err, opened = io.StringIO(), io.StringIO(), []

    def opener(model_dir, dtype, device):
        opened.append((model_dir, dtype, device))
        opener.model = FakeModel()
        return opener.model
    rc = cli.main(argv, out=out, err=err, opener=opener)
    return rc, out.getvalue(), err.getvalue(), opened, getattr(opener, "model", None)


def test_run_flags_reach_the_policy():
    rc, out, err, opened, model = run(["run", "--prompt", "5, 17 3", "--max-tokens", "4", "--temp",
                                       "0.7", "--top-k", "40", "--top-p", "0.9", "--repeat-penalty",
                                       "1.1", "--seed", "9", "--precision", "f32", "--context", "64",
                                       "/models/x"])
    assert rc == 0 and out.split() == ["100", "101", "102", "103"]
    assert opened == [("/models/x", "float32", "cuda:0")]
    prompt, pol = model.sessions[0].calls[0]
    assert prompt == [5, 17, 3] and model.sessions[0].context == 64
    assert (pol.temperature, pol.top_k, pol.top_p, pol.repetition_penalty, pol.seed,
            pol.max_tokens) == (0.7, 40, 0.9, 1.1, 9, 4)
    assert "4 generated" in err


def test_defaults_are_the_references():
    a = cli.run_parser().parse_args(["m"])
    assert (a.max_tokens, a.temp, a.top_k, a.top_p, a.repeat_penalty, a.seed, a.precision,
            a.context, a.device) == (128, 0.0, 0, 0.0, 1.0, 0, "auto", 4096, "auto")
    b = cli.bench_parser().parse_args(["m"])
    assert (b.tokens, b.prompt_tokens, b.batch, b.warmup, b.json) == (128, 128, "1", 8, "")
    assert (a.page_size, a.kv_pages, a.stop_ids, a.prompt, a.prompt_len) == (16, 0, "auto", None, 0)


def test_stop_ids_page_size_and_several_prompts():
    """What goes beyond the reference's flags: stop ids (the model folder's by default), the
    page size, and several prompts, which run together through the scheduler."""
    rc, out, err, _, model = run(["run", "--max-tokens", "2", "--page-size", "8", "m"])
    assert rc == 0 and model.sessions[0].kw == {"page_size": 8, "stop_ids": [7, 9]}
    assert model.sessions[0].calls[0][0] == [1, 2, 3, 4, 5, 6, 7, 8]
    rc, out, err, _, model = run(["run", "--max-tokens", "2", "--stop-ids", "3,4", "m"])
    assert model.sessions[0].kw["stop_ids"] == [3, 4]
    rc, out, err, _, model = run(["run", "--max-tokens", "2", "--stop-ids", "none", "m"])
    assert model.sessions[0].kw["stop_ids"] == []
    rc, out, err, _, model = run(["run", "--prompt", "1 2", "--prompt", "3,4,5", "--max-tokens", "3",
                                  "--seed", "5", "--kv-pages", "40", "--context", "64", "m"])
    assert rc == 0 and not model.sessions
    prompts, policies, kw = model.generated[0]
    assert prompts == [[1, 2], [3, 4, 5]] and [p.seed for p in policies] == [5, 6]
    assert kw == {"slots": 2, "pool_tokens": 640, "page_size": 16, "stop_ids": [7, 9]}
    assert out.splitlines() == ["200 200 200", "201 201 201"] and "2 prompts" in err
    rc, out, err, _, model = run(["run", "--prompt-len", "11", "--max-tokens", "1", "m"])
    assert rc == 0 and len(model.sessions[0].calls[0][0]) == 11


@pytest.mark.parametrize("argv,needle", [
    (["run", "--max-tokens", "0", "m"], "max-tokens"),
    (["run", "--max-tokens", "100", "--context", "50", "m"], "more than the --context"),
    (["run", "--prompt", "hello world", "m"], "token ids"),
    (["run", "--prompt", " ", "m"], "empty"),
    (["run", "--precision", "int4", "m"], "bf16, f32 or auto"),
    (["run", "--device", "metal", "m"], "no other device"),
    (["run", "--top-k", "500", "m"], "top_k"),
    (["run", "--temp", "-1", "m"], "temperature"),
    (["bench", "--tokens", "100", "--prompt-tokens", "100", "--context", "150", "m"], "more than"),
    (["bench", "--warmup", "-1", "m"], "warmup"),
    (["bench", "--batch", "0", "m"], "batch"),
    (["bench", "--batch", "1,x", "m"], "batch"),
    (["run", "--stop-ids", "eos", "m"], "stop-ids"),
    (["run", "--prompt", "1", "--prompt-len", "4", "m"], "prompt-len"),
    (["run", "--config", "c.json", "m"], "go together"),
    (["run"], "<model-dir> is needed"),
    (["run", "--prompt", "1 2 3", "--prompt", "4", "--max-tokens", "60", "--context", "62", "m"], "exceed"),
])
def test_usage_errors_name_the_flag(argv, needle):
    rc, out, err, opened, _ = run(argv)
    assert rc == 2 and needle in err


def test_unknown_command_and_help():
    rc, out, err, _, _ = run(["serve"])
    assert rc == 2 and "unknown command" in err
    rc, out, err, _, _ = run(["--help"])
    assert rc == 0 and "tgo run" in out
    rc, out, err, _, _ = run([])
    assert rc == 2


def test_policy_refusals_and_draw_stream():
    Policy().check(10)
    for bad in (Policy(temperature=float("nan")), Policy(top_k=129), Policy(top_p=1.5),
                Policy(repetition_penalty=-1), Policy(penalty_window=-2),
                Policy(logit_bias={10: 1.0}), Policy(logit_bias={1: float("inf")}),
                Policy(presence_penalty=float("nan")), Policy(max_tokens=-1),
                Policy(top_logprobs=3), Policy(logprobs=True, top_logprobs=129),
                Policy(logprobs=True, top_logprobs=-1)):
        with pytest.raises(ValueError):
            bad.check(10)
    Policy(logit_bias={1: float("-inf")}).check(10)        # banning a token is allowed
    Policy(logprobs=True, top_logprobs=128).check(10)
    a, b = DrawStream(5), DrawStream(5)
    xs = [a.next() for _ in range(100)]
    assert xs == [b.next() for _ in range(100)] and xs != [DrawStream(6).next() for _ in range(100)]
    assert all(0 <= x < 1 for x in xs) and 0.3 < sum(xs) / 100 < 0.7
