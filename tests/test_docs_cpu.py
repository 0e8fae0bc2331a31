"""The guides under ``docs/`` stay true: every Python block that starts with ``# runnable`` is executed (CPU), every
relative link and every repository path a guide names exists."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = os.path.join(ROOT, "docs")
GUIDES = sorted(f for f in os.listdir(DOCS) if f.endswith(".md"))


def _blocks(text):
    return [m.group(1) for m in re.finditer(r"```python\n(.*?)```", text, re.S)]


@pytest.mark.parametrize("guide", GUIDES)
def test_runnable_blocks_execute(guide, tmp_path, monkeypatch):
    text = open(os.path.join(DOCS, guide)).read()
    monkeypatch.chdir(tmp_path)                      # blocks that write files write into a scratch directory
    ran = 0
    env = {"__name__": "__docs__"}                   # one namespace per guide: later blocks may use earlier names
    for code in _blocks(text):
        if code.lstrip().startswith("# runnable"):
            exec(compile(code, f"{guide}:block{ran}", "exec"), env)
            ran += 1
    assert ran > 0 or guide in ("README.md", "faq.md", "installation.md", "profiling_benchmarks.md"), f"{guide} has no runnable block"


@pytest.mark.parametrize("guide", GUIDES)
def test_links_and_named_paths_exist(guide):
    text = open(os.path.join(DOCS, guide)).read()
    for target in re.findall(r"\]\(([^)#]+\.md)\)", text):
        assert os.path.exists(os.path.join(DOCS, target)), f"{guide} links to missing {target}"
    for path in re.findall(r"`((?:sneppx_alg_b200|examples|tests|profiles|sneppx|SneppX_ALG)/[A-Za-z0-9_./-]+)`", text):
        assert os.path.exists(os.path.join(ROOT, path)), f"{guide} names missing {path}"
