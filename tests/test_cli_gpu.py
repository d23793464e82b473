"""The command line as a user runs it (a subprocess): ids in, ids out; several prompts through
the scheduler with a cache so small that requests are preempted, and the ids must be those each
prompt gets alone (the reference's parser: qwen-infer/src/main.rs:76-138)."""
import os
import re
import subprocess
import sys

import pytest

from tiny import make_folder, random_ids

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "bin", "qwen-infer")


def run_cli(*args):
    proc = subprocess.run([sys.executable, CLI, *args], capture_output=True, text=True, timeout=600)
    return proc.returncode, proc.stdout, proc.stderr


def test_several_prompts_on_a_small_cache_print_the_ids_of_each_alone(tmp_path_factory):
    folder, config, page = make_folder(tmp_path_factory, "b")
    prompts = [random_ids(n, config.vocab_size, 60 + n) for n in (9, 30, 17)]
    as_text = [",".join(str(t) for t in p) for p in prompts]
    alone = []
    for text in as_text:
        rc, out, err = run_cli("--model", folder, "--dtype", "float32", "--max-tokens", "14", "--ids", text)
        assert rc == 0, err
        alone.append(out.strip())
        assert "generated ids:" in err and "stop: MAX_TOKENS" in err and "tok/s" in err
    # room for about half of the three at their final length
    pages = max(sum(-(-(len(p) + 14) // page) for p in prompts) // 2, -(-(30 + 14) // page) + 1)
    several = []
    for flag in ("--ids",):
        for text in as_text:
            several += [flag, text]
    rc, out, err = run_cli("--model", folder, "--dtype", "float32", "--max-tokens", "14", *several,
                           "--num-pages", str(pages), "--page-size", str(page),
                           "--max-batch-size", "3", "--token-budget", "16")
    assert rc == 0, err
    assert out.strip().splitlines() == alone
    found = re.search(r"preemptions (\d+)", err)
    assert found and int(found.group(1)) > 0, err
    assert "[2] generated ids:" in err and "most running 3" in err
    # one prompt that no cache of this size can hold fails with a message, the others run
    rc, out, err = run_cli("--model", folder, "--dtype", "float32", "--max-tokens", "4",
                           "--ids", ",".join(["5"] * 100), "--ids", "1,2,3",
                           "--num-pages", "4", "--page-size", str(page))
    assert rc == 1 and "[0] error:" in err and "[1] generated ids:" in err


def test_usage_errors():
    rc, out, err = run_cli()
    assert rc == 1 and "usage: qwen-infer" in err
    rc, out, err = run_cli("--nope")
    assert rc == 2 and "unknown argument --nope" in err
