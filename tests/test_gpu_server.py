"""The public path on a B200: a quantised checkpoint directory on disk -> loader (native reader threads, manifest)
-> engine on the GPU -> scheduler with captured decode steps -> HTTP/SSE server on loopback."""
import json
import threading
import urllib.request

import pytest
import torch

from vade_b200.checkpoint.synth import write_checkpoint
from vade_b200.config import QuantConfig, small_gpu_config
from vade_b200.runtime.build import load_engine
from vade_b200.runtime.scheduler import Scheduler, SchedulerConfig
from vade_b200.serve.http import ApiServer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("ckpt_gpu"))
    cfg = small_gpu_config()
    write_checkpoint(cfg, root, seed=0)
    eng, tok, receipt = load_engine(root, device="cuda", slots=10, max_seq=512, prefill_chunk=128)
    sched = Scheduler(eng, SchedulerConfig(prefill_slice=128, max_active=8), eos_id=tok.eos_id, detokenize=tok.decode)
    api = ApiServer(sched, tok, "small", {"checkpoint": receipt["fingerprint"], "world": 1})
    port = api.start()
    yield api, port, eng, sched
    api.stop()


def _post(port, path, obj, stream=False):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", json.dumps(obj).encode(), {"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=180) as r:
        raw = r.read().decode()
    if not stream:
        return json.loads(raw)
    return [json.loads(l[6:]) for l in raw.split("\n") if l.startswith("data: ") and l != "data: [DONE]"]


def _ids(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 8000, (n,), generator=g).tolist()


def test_server_on_gpu_matches_the_engine_streams_and_batches(server):
    api, port, eng, sched = server
    prompt = _ids(90, 1)
    body = {"prompt": prompt, "max_tokens": 16, "ignore_eos": True, "draft": "plain"}
    got = _post(port, "/v1/completions", body)["choices"][0]["token_ids"]
    assert len(got) == 16
    assert got == eng.generate(prompt, 16).generated, "the served ids differ from the engine's own generation"
    chunks = _post(port, "/v1/completions", {**body, "stream": True}, stream=True)
    assert [c["choices"][0]["token_id"] for c in chunks if c["choices"] and "token_id" in c["choices"][0]] == got
    # concurrent chats (captured steps of widths 2..8) give each chat its solo ids; drafting keeps them too
    prompts = [_ids(40 + 17 * i, 10 + i) for i in range(6)]
    solo = [_post(port, "/v1/completions", {"prompt": p, "max_tokens": 10, "ignore_eos": True, "draft": "plain"})["choices"][0]["token_ids"]
            for p in prompts]
    res = [None] * len(prompts)

    def run(i):
        res[i] = _post(port, "/v1/completions", {"prompt": prompts[i], "max_tokens": 10, "ignore_eos": True, "draft": "plain"})["choices"][0]["token_ids"]
    th = [threading.Thread(target=run, args=(i,)) for i in range(len(prompts))]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert res == solo
    drafted = _post(port, "/v1/completions", {**body, "draft": "strict", "mtp_depth": 3})
    assert drafted["choices"][0]["token_ids"] == got
    sampled = {"prompt": prompt, "max_tokens": 12, "ignore_eos": True, "temperature": 0.8, "top_k": 40, "top_p": 0.9, "seed": 7}
    assert _post(port, "/v1/completions", sampled)["choices"][0]["token_ids"] == _post(port, "/v1/completions", sampled)["choices"][0]["token_ids"]
    health = json.loads(urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=30).read())
    assert health["status"] == "ok"
    assert sched.pool is not None and sched.pool.replays > 0
    eng.model.ops.check_status()
