"""S5 extensions: data-poisoning defence and output-policy ("RLHF safety") scoring.

``PoisonDetector`` models clean training samples by per-feature mean / standard deviation (Welford updates, so it can
keep learning one sample at a time), scores a sample by its root-mean-square z-score, and flags outliers above a
threshold that can be set by hand or from the clean data's own score quantile. Around it: batch checks, ensemble
voting, k-fold cross-validation of the false-positive rate, per-feature importance (how much each feature separates
flagged from unflagged samples), label-flip screening with nearest neighbours, and model export / import.
``SafetyPolicyEngine`` holds weighted policies (keyword / regular expression / length / repetition / custom
callable), scores a (prompt, answer) pair into helpfulness / harmlessness / honesty components, lists violations,
writes a critique, produces a refusal, and rewrites an answer with the offending spans redacted.
Reference modules of the same purpose: security/ai/data_poisoning_defense.c (train / score / is_outlier /
incremental update / ensemble / cross-validate / feature importance / adaptive threshold / export) and
security/ai/rlhf_safety.c (policies, score, check, refusal, critique, correct, stats).
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np


# ----------------------------------------------------------------------------------------------- poisoning
class PoisonDetector:
    def __init__(self, feature_count: int, threshold: float = 3.0):
        self.d, self.threshold = feature_count, threshold
        self.reset()

    def reset(self) -> None:
        self.n = 0
        self.mean = np.zeros(self.d)
        self.m2 = np.zeros(self.d)
        self.checked = self.flagged = 0

    @property
    def std(self) -> np.ndarray:
        return np.sqrt(self.m2 / max(self.n - 1, 1)) if self.n > 1 else np.ones(self.d)

    def train(self, samples) -> None:
        x = np.asarray(samples, dtype=np.float64).reshape(-1, self.d)
        self.n = x.shape[0]
        self.mean = x.mean(0)
        self.m2 = ((x - self.mean) ** 2).sum(0)

    def update(self, sample, learning_rate: Optional[float] = None) -> None:
        """One more clean sample: exact running statistics, or an exponential moving average when a rate is given
        (tracks slow drift of the data distribution)."""
        x = np.asarray(sample, dtype=np.float64).reshape(self.d)
        if learning_rate is not None and self.n > 1:
            var = self.m2 / (self.n - 1)
            delta = x - self.mean
            self.mean = self.mean + learning_rate * delta
            var = (1 - learning_rate) * (var + learning_rate * delta * delta)
            self.m2 = var * (self.n - 1)
            return
        self.n += 1
        delta = x - self.mean
        self.mean = self.mean + delta / self.n
        self.m2 = self.m2 + delta * (x - self.mean)

    def score(self, sample) -> float:
        z = (np.asarray(sample, dtype=np.float64).reshape(self.d) - self.mean) / np.maximum(self.std, 1e-12)
        return float(np.sqrt(np.mean(z * z)))

    def scores(self, samples) -> np.ndarray:
        x = np.asarray(samples, dtype=np.float64).reshape(-1, self.d)
        z = (x - self.mean) / np.maximum(self.std, 1e-12)
        return np.sqrt((z * z).mean(1))

    def is_outlier(self, sample) -> bool:
        self.checked += 1
        out = self.score(sample) > self.threshold
        self.flagged += int(out)
        return out

    def batch_check(self, samples) -> np.ndarray:
        s = self.scores(samples) > self.threshold
        self.checked += s.size
        self.flagged += int(s.sum())
        return s

    def find_outliers(self, samples) -> List[int]:
        return [int(i) for i in np.nonzero(self.scores(samples) > self.threshold)[0]]

    def adaptive_threshold(self, clean_samples, sensitivity: float = 0.99) -> float:
        """Threshold = the ``sensitivity`` quantile of the clean data's own scores (that fraction of clean data passes)."""
        self.threshold = float(np.quantile(self.scores(clean_samples), sensitivity))
        return self.threshold

    def stats(self) -> dict:
        return {"samples": self.n, "checked": self.checked, "outlier_rate": self.flagged / max(self.checked, 1)}

    def feature_importance(self, samples) -> np.ndarray:
        """Per feature: mean |z| of flagged samples minus mean |z| of the rest, normalised to sum to 1 (zeros if nothing
        is flagged)."""
        x = np.asarray(samples, dtype=np.float64).reshape(-1, self.d)
        z = np.abs((x - self.mean) / np.maximum(self.std, 1e-12))
        flag = self.scores(x) > self.threshold
        if not flag.any() or flag.all():
            return np.zeros(self.d)
        gap = np.maximum(z[flag].mean(0) - z[~flag].mean(0), 0)
        return gap / gap.sum() if gap.sum() > 0 else gap

    def export_model(self) -> dict:
        return {"mean": self.mean.tolist(), "std": self.std.tolist(), "n": self.n, "threshold": self.threshold}

    @classmethod
    def import_model(cls, m: dict) -> "PoisonDetector":
        pd = cls(len(m["mean"]), m["threshold"])
        pd.n = int(m["n"])
        pd.mean = np.asarray(m["mean"], dtype=np.float64)
        pd.m2 = np.asarray(m["std"], dtype=np.float64) ** 2 * max(pd.n - 1, 1)
        return pd


def ensemble_is_outlier(detectors: Sequence[PoisonDetector], sample, quorum: Optional[int] = None) -> bool:
    votes = sum(d.score(sample) > d.threshold for d in detectors)
    return votes >= (quorum if quorum is not None else len(detectors) // 2 + 1)


def cross_validate(samples, folds: int = 5, threshold: float = 3.0, seed: int = 0) -> float:
    """Mean fraction of held-out CLEAN samples that a detector trained on the other folds accepts."""
    x = np.asarray(samples, dtype=np.float64)
    idx = np.random.default_rng(seed).permutation(len(x))
    acc = []
    for f in range(folds):
        test = idx[f::folds]
        train = np.setdiff1d(idx, test)
        pd = PoisonDetector(x.shape[1], threshold)
        pd.train(x[train])
        acc.append(float((pd.scores(x[test]) <= threshold).mean()))
    return float(np.mean(acc))


def label_flip_suspects(features, labels, k: int = 5) -> List[int]:
    """Samples whose label disagrees with the majority label of their k nearest neighbours (label-flipping attacks)."""
    x = np.asarray(features, dtype=np.float64)
    y = np.asarray(labels)
    d2 = ((x[:, None, :] - x[None, :, :]) ** 2).sum(-1)
    np.fill_diagonal(d2, np.inf)
    out = []
    for i in range(len(x)):
        nn = np.argsort(d2[i])[:k]
        vals, counts = np.unique(y[nn], return_counts=True)
        if vals[np.argmax(counts)] != y[i] and counts.max() > k // 2:
            out.append(i)
    return out


# ----------------------------------------------------------------------------------------------- output policies
@dataclass
class Policy:
    name: str
    weight: float
    kind: str                 # keyword | regex | max_length | repetition | custom
    pattern: object = None
    threshold: float = 0.0
    dimension: str = "harmlessness"      # which score component a violation lowers
    id: int = 0


@dataclass
class Violation:
    policy: str
    severity: float
    span: Tuple[int, int]
    excerpt: str


@dataclass
class SafetyScore:
    helpfulness: float
    harmlessness: float
    honesty: float
    overall: float
    violations: List[Violation] = field(default_factory=list)

    @property
    def acceptable(self) -> bool:
        return self.overall >= 0.5 and self.harmlessness >= 0.5


DEFAULT_POLICIES = [
    ("violence", 1.0, "regex", r"\b(how to (build|make) (a )?(bomb|explosive)|kill (him|her|them|someone))\b", "harmlessness"),
    ("self_harm", 1.0, "regex", r"\b(ways to (hurt|harm) (yourself|myself)|commit suicide)\b", "harmlessness"),
    ("malware", 0.9, "regex", r"\b(ransomware|keylogger|reverse shell) (source|code|payload)\b", "harmlessness"),
    ("credentials", 0.8, "regex", r"(password|api[_ ]?key|secret)\s*[:=]\s*\S{6,}", "harmlessness"),
    ("overclaim", 0.5, "regex", r"\b(i am (100% )?certain|guaranteed to|cannot be wrong)\b", "honesty"),
    ("fabricated_citation", 0.5, "regex", r"\(\s*(Smith|Doe|Johnson) et al\.,? (19|20)\d\d\s*\)", "honesty"),
    ("too_long", 0.3, "max_length", None, "helpfulness"),
    ("repetition", 0.4, "repetition", None, "helpfulness"),
]


class SafetyPolicyEngine:
    def __init__(self, defaults: bool = True, refusal_threshold: float = 0.5, max_length: int = 8000):
        self.policies: Dict[int, Policy] = {}
        self._next = 1
        self.refusal_threshold, self.max_length = refusal_threshold, max_length
        self.stats = {"scored": 0, "refused": 0, "violations": 0, "corrected": 0}
        if defaults:
            self.add_default_policies()

    def add_policy(self, name, weight, kind, pattern=None, threshold=0.0, dimension="harmlessness") -> int:
        if kind not in ("keyword", "regex", "max_length", "repetition", "custom"):
            raise ValueError(f"unknown policy kind {kind!r}")
        if kind == "regex":
            pattern = re.compile(pattern, re.I)
        p = Policy(name, float(weight), kind, pattern, threshold, dimension, self._next)
        self.policies[p.id] = p
        self._next += 1
        return p.id

    def remove_policy(self, pid: int) -> bool:
        return self.policies.pop(pid, None) is not None

    def add_default_policies(self) -> int:
        for name, w, kind, pat, dim in DEFAULT_POLICIES:
            self.add_policy(name, w, kind, pat, self.max_length if kind == "max_length" else 0.3, dim)
        return len(DEFAULT_POLICIES)

    def check_policies(self, text: str) -> List[Violation]:
        out = []
        for p in self.policies.values():
            if p.kind == "keyword":
                for m in re.finditer(re.escape(str(p.pattern)), text, re.I):
                    out.append(Violation(p.name, p.weight, m.span(), text[m.start():m.end()]))
            elif p.kind == "regex":
                for m in p.pattern.finditer(text):
                    out.append(Violation(p.name, p.weight, m.span(), text[m.start():m.end()][:80]))
            elif p.kind == "max_length" and len(text) > p.threshold:
                out.append(Violation(p.name, p.weight, (int(p.threshold), len(text)), f"{len(text)} characters"))
            elif p.kind == "repetition":
                words = text.lower().split()
                if len(words) >= 20:
                    grams = [" ".join(words[i:i + 4]) for i in range(len(words) - 3)]
                    rep = 1.0 - len(set(grams)) / len(grams)
                    if rep > p.threshold:
                        out.append(Violation(p.name, p.weight * rep, (0, len(text)), f"{rep:.0%} repeated 4-grams"))
            elif p.kind == "custom":
                r = p.pattern(text)
                if r:
                    out.append(Violation(p.name, p.weight * (float(r) if not isinstance(r, bool) else 1.0), (0, len(text)), ""))
        return out

    def score(self, prompt: str, answer: str) -> SafetyScore:
        self.stats["scored"] += 1
        v = self.check_policies(answer)
        self.stats["violations"] += len(v)
        dims = {"helpfulness": 1.0, "harmlessness": 1.0, "honesty": 1.0}
        by_name = {p.name: p for p in self.policies.values()}
        for viol in v:
            d = by_name[viol.policy].dimension
            dims[d] = max(0.0, dims[d] - viol.severity * 0.6)
        # helpfulness: an empty answer or one that shares no content word with the prompt helps nobody
        pw = {w for w in re.findall(r"[a-z]{4,}", prompt.lower())}
        aw = {w for w in re.findall(r"[a-z]{4,}", answer.lower())}
        if not answer.strip():
            dims["helpfulness"] = 0.0
        elif pw and not (pw & aw):
            dims["helpfulness"] = min(dims["helpfulness"], 0.5)
        overall = 0.3 * dims["helpfulness"] + 0.5 * dims["harmlessness"] + 0.2 * dims["honesty"]
        return SafetyScore(dims["helpfulness"], dims["harmlessness"], dims["honesty"], overall, v)

    def generate_refusal(self, score: SafetyScore) -> str:
        self.stats["refused"] += 1
        topics = sorted({v.policy.replace("_", " ") for v in score.violations if v.severity >= 0.5})
        about = f" (it touches on: {', '.join(topics)})" if topics else ""
        return f"I can't help with that request{about}. I can help with a safer or more general version of it."

    def generate_critique(self, answer: str) -> str:
        v = self.check_policies(answer)
        if not v:
            return "No policy concerns found."
        return "\n".join(f"- {x.policy}: severity {x.severity:.2f} at characters {x.span[0]}-{x.span[1]}"
                         + (f" ({x.excerpt!r})" if x.excerpt else "") for x in v)

    def correct_output(self, answer: str) -> str:
        """The answer with every span-level violation replaced by a marker and an over-long tail cut."""
        spans = sorted((x.span for x in self.check_policies(answer)
                        if x.span != (0, len(answer)) and x.policy != "too_long"), reverse=True)
        out = answer
        for a, b in spans:
            out = out[:a] + "[removed]" + out[b:]
        if len(out) > self.max_length:
            out = out[: self.max_length].rstrip() + " [truncated]"
        if out != answer:
            self.stats["corrected"] += 1
        return out

    def respond(self, prompt: str, answer: str) -> Tuple[str, SafetyScore]:
        """What the serving path returns: the answer, a corrected answer, or a refusal."""
        s = self.score(prompt, answer)
        if s.harmlessness < self.refusal_threshold:
            return self.generate_refusal(s), s
        return (self.correct_output(answer) if s.violations else answer), s
