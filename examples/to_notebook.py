"""Turns an example script into a Jupyter notebook (nbformat 4, no dependency on the ``nbformat`` package): the module
docstring becomes the opening Markdown cell, the imports one code cell, every top-level definition its own cell, and a
last cell calls ``main()``.

    python examples/to_notebook.py examples/ex_06_llama_train_generate_checkpoint.py            # writes examples/notebooks/<name>.ipynb
    python examples/to_notebook.py --all
"""
import ast
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "notebooks")


def _cell(kind: str, text: str) -> dict:
    lines = text.strip("\n").split("\n")
    source = [l + "\n" for l in lines[:-1]] + [lines[-1]]
    if kind == "markdown":
        return {"cell_type": "markdown", "metadata": {}, "source": source}
    return {"cell_type": "code", "execution_count": None, "metadata": {}, "outputs": [], "source": source}


def convert(path: str) -> dict:
    src = open(path).read()
    tree = ast.parse(src)
    lines = src.split("\n")
    title = os.path.splitext(os.path.basename(path))[0]
    cells = [_cell("markdown", f"# {title}\n\n{ast.get_docstring(tree) or ''}\n\nRun from the `examples/` directory of a checkout "
                               "(the first import makes the package importable from there).")]
    body = tree.body[1:] if ast.get_docstring(tree) else tree.body
    imports, rest = [], []
    for node in body:
        (imports if isinstance(node, (ast.Import, ast.ImportFrom)) and not rest else rest).append(node)

    def text(nodes):
        start = min(getattr(n, "decorator_list", None) and n.decorator_list[0].lineno or n.lineno for n in nodes)
        return "\n".join(lines[start - 1:max(n.end_lineno for n in nodes)])

    if imports:
        cells.append(_cell("code", text(imports)))
    for node in rest:
        if isinstance(node, ast.If) and "__name__" in ast.dump(node.test):
            continue                                         # the script entry point; the notebook calls main() itself
        cells.append(_cell("code", text([node])))
    cells.append(_cell("code", "result = main()\nresult"))
    return {"cells": cells, "metadata": {"kernelspec": {"display_name": "Python 3", "language": "python", "name": "python3"},
                                         "language_info": {"name": "python"}}, "nbformat": 4, "nbformat_minor": 5}


def write(path: str, out_dir: str = OUT) -> str:
    os.makedirs(out_dir, exist_ok=True)
    dest = os.path.join(out_dir, os.path.splitext(os.path.basename(path))[0] + ".ipynb")
    with open(dest, "w") as f:
        json.dump(convert(path), f, indent=1)
        f.write("\n")
    return dest


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if argv == ["--all"]:
        # every example except the one that spawns worker processes (they cannot import functions defined in a notebook)
        argv = sorted(os.path.join(HERE, f) for f in os.listdir(HERE)
                      if f.startswith("ex_") and f.endswith(".py") and not f.startswith("ex_10_"))
    if not argv:
        print(__doc__)
        return []
    return [write(p) for p in argv]


if __name__ == "__main__":
    for p in main():
        print(p)
