"""S5 extensions: defences around a served or trained model beyond the prompt filter and the output verifier.

* inputs: ``SemanticInjectionDetector`` (nearest known attack in a hashed n-gram embedding), ``JailbreakDetector``
  (weighted phrase patterns, also applied to decoded payloads), ``decode_layers`` / ``scan_encoded`` (base64 / hex /
  rot13 / URL-escape wrappers, peeled recursively), ``PromptPolicy`` (allow / deny / require rules);
* outputs: ``token_anomaly_score`` / ``perplexity`` (how unlikely the sampled tokens were under the model),
  ``DataExtractionGuard`` (secrets and personal data in generated text), ``factuality_score`` (n-gram support of a
  statement by a reference text);
* training data: ``sanitize_training_text`` (e-mail, phone, IP, URL, national-id redaction);
* privacy: ``ModelInversionDefense`` (per-step gradient clipping + Gaussian noise), ``membership_inference_defense``
  (logit clamp + Laplace noise), ``adversarial_smooth`` (randomised-smoothing average of a classifier);
* fairness: ``BiasMetrics`` (demographic parity, equalised odds, disparate impact).

Reference behaviour: security/ai/s5_extensions.c (function families ``semantic_injection_*``, ``ml_jailbreak_*``,
``encoded_attack_*``, ``token_anomaly_*``, ``model_inversion_*``, ``membership_inference_*``, ``data_extraction_*``,
``training_sanitize_*``, ``adversarial_smooth*``, ``factuality_score*``, ``bias_measure*``, ``prompt_policy_*``).
Weight watermarks are in ``security/model_watermark.py``.
"""
from __future__ import annotations

import base64
import binascii
import codecs
import hashlib
import math
import re
import urllib.parse
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------------------------------ text embedding
def text_embedding(text: str, dim: int = 64, n: int = 3) -> torch.Tensor:
    """Unit-norm bag of hashed character n-grams of the lower-cased, whitespace-collapsed text (signed hashing, so
    collisions cancel in expectation). Near-duplicate and lightly reworded texts land close in cosine distance."""
    t = re.sub(r"\s+", " ", text.lower()).strip()
    v = torch.zeros(dim, dtype=torch.float64)
    for i in range(max(1, len(t) - n + 1)):
        h = int.from_bytes(hashlib.blake2b(t[i:i + n].encode(), digest_size=8).digest(), "big")
        v[h % dim] += 1.0 if (h >> 32) & 1 else -1.0
    nrm = v.norm()
    return v / nrm if nrm > 0 else v


class SemanticInjectionDetector:
    """Keeps embeddings of known injection prompts; ``score`` is the highest cosine similarity of a new prompt to any
    of them and ``is_attack`` compares it with ``threshold``."""

    def __init__(self, threshold: float = 0.75, dim: int = 64, capacity: int = 4096):
        self.threshold, self.dim, self.capacity = float(threshold), dim, capacity
        self._texts: List[str] = []
        self._bank = torch.zeros(0, dim, dtype=torch.float64)
        self.queries = self.hits = 0

    def add_attack(self, text: str) -> int:
        if len(self._texts) >= self.capacity:
            raise OverflowError("attack bank is full")
        self._texts.append(text)
        self._bank = torch.cat([self._bank, text_embedding(text, self.dim)[None]])
        return len(self._texts) - 1

    def add_attacks(self, texts: Iterable[str]) -> int:
        return sum(1 for t in texts if self.add_attack(t) >= 0)

    def remove_attack(self, index: int) -> bool:
        if not 0 <= index < len(self._texts):
            return False
        del self._texts[index]
        self._bank = torch.cat([self._bank[:index], self._bank[index + 1:]])
        return True

    def clear(self) -> None:
        self._texts, self._bank = [], torch.zeros(0, self.dim, dtype=torch.float64)

    def __len__(self) -> int:
        return len(self._texts)

    def find_closest(self, text: str) -> Tuple[int, float]:
        """(index of the nearest stored attack, cosine similarity); (-1, 0.0) with an empty bank."""
        if not self._texts:
            return -1, 0.0
        sims = self._bank @ text_embedding(text, self.dim)
        i = int(sims.argmax())
        return i, float(sims[i])

    def score(self, text: str) -> float:
        return max(0.0, self.find_closest(text)[1])

    def is_attack(self, text: str) -> bool:
        self.queries += 1
        hit = self.score(text) >= self.threshold
        self.hits += int(hit)
        return hit

    def stats(self) -> dict:
        return {"attacks": len(self), "queries": self.queries, "hits": self.hits, "threshold": self.threshold}


# ------------------------------------------------------------------------------------------------ encoded payloads
_B64 = re.compile(r"(?<![A-Za-z0-9+/=_-])[A-Za-z0-9+/_-]{16,}={0,2}(?![A-Za-z0-9+/=_-])")
_HEX = re.compile(r"(?<![0-9A-Fa-f])(?:0x)?((?:[0-9A-Fa-f]{2}){8,})(?![0-9A-Fa-f])")
_PCT = re.compile(r"(?:%[0-9A-Fa-f]{2}){3,}")


def _printable(b: bytes) -> Optional[str]:
    try:
        s = b.decode("utf-8")
    except UnicodeDecodeError:
        return None
    good = sum(ch.isprintable() or ch in "\n\t" for ch in s)
    return s if s and good / len(s) > 0.9 else None


def detect_encoding(s: str) -> str:
    """"base64" / "hex" / "url" / "none" for a string that is, as a whole, one such encoding of printable text."""
    t = s.strip()
    if len(t) >= 8 and _HEX.fullmatch(t) and _printable(bytes.fromhex(t[2:] if t.lower().startswith("0x") else t)):
        return "hex"
    if len(t) >= 8 and len(t) % 4 != 1 and _B64.fullmatch(t) and decode_base64(t) is not None:
        return "base64"
    if _PCT.search(t):
        return "url"
    return "none"


def decode_base64(s: str) -> Optional[str]:
    t = s.strip().replace("-", "+").replace("_", "/")
    try:
        return _printable(base64.b64decode(t + "=" * (-len(t) % 4), validate=True))
    except (binascii.Error, ValueError):
        return None


def decode_hex(s: str) -> Optional[str]:
    t = s.strip()
    t = t[2:] if t.lower().startswith("0x") else t
    try:
        return _printable(bytes.fromhex(t))
    except ValueError:
        return None


def decode_rot13(s: str) -> str:
    return codecs.decode(s, "rot13")


def decode_layers(text: str, max_depth: int = 4) -> List[Tuple[str, str]]:
    """Every payload found by peeling base64 / hex / URL-escape runs out of ``text``, recursively up to ``max_depth``
    layers, as (encoding chain such as "base64>hex", decoded text). rot13 of the whole text is offered at depth 1
    only (it is its own inverse and matches everything)."""
    found: List[Tuple[str, str]] = []
    seen = set()

    def walk(t: str, chain: str, depth: int):
        if depth >= max_depth:
            return
        cands: List[Tuple[str, str]] = []
        for m in _B64.finditer(t):
            d = decode_base64(m.group(0))
            if d is not None:
                cands.append(("base64", d))
        for m in _HEX.finditer(t):
            d = decode_hex(m.group(1))
            if d is not None:
                cands.append(("hex", d))
        if _PCT.search(t):
            cands.append(("url", urllib.parse.unquote(t)))
        for enc, d in cands:
            if d in seen or d == t:
                continue
            seen.add(d)
            c = f"{chain}>{enc}" if chain else enc
            found.append((c, d))
            walk(d, c, depth + 1)

    walk(text, "", 0)
    if max_depth > 0:
        r = decode_rot13(text)
        if r not in seen and r != text:
            found.append(("rot13", r))
    return found


# ------------------------------------------------------------------------------------------------ jailbreak phrases
_DEFAULT_JAILBREAK = (
    (r"ignore (all |any )?(the )?(previous|prior|above|earlier) (instructions|rules|prompts?)", 0.9),
    (r"disregard (all |any )?(the )?(previous|prior|above|system) ", 0.8),
    (r"you are (now )?(dan|in developer mode|an? unrestricted|no longer bound)", 0.9),
    (r"pretend (that )?you (have no|are not bound by|can ignore) ", 0.7),
    (r"(reveal|print|show|repeat) (me )?(your |the )?(system|hidden|initial) (prompt|instructions)", 0.8),
    (r"without (any )?(ethical|moral|safety) (guidelines|restrictions|filters?)", 0.7),
    (r"do anything now", 0.8),
    (r"jailbr(eak|oken)", 0.6),
    (r"respond only as .{0,40}(evil|unfiltered|uncensored)", 0.7),
)


class JailbreakDetector:
    """Weighted phrase patterns; the confidence of a text is 1 - prod(1 - w) over the patterns that match, taken over
    the text itself and every payload ``decode_layers`` finds in it."""

    def __init__(self, threshold: float = 0.6, patterns: Optional[Sequence[Tuple[str, float]]] = None):
        self.threshold = float(threshold)
        self._patterns: List[Tuple[str, float, re.Pattern]] = []
        for p, w in (_DEFAULT_JAILBREAK if patterns is None else patterns):
            self.add_pattern(p, w)

    def add_pattern(self, pattern: str, weight: float = 0.7) -> None:
        self._patterns.append((pattern, float(weight), re.compile(pattern, re.IGNORECASE)))

    def remove_pattern(self, pattern: str) -> bool:
        n = len(self._patterns)
        self._patterns = [p for p in self._patterns if p[0] != pattern]
        return len(self._patterns) < n

    def patterns(self) -> List[str]:
        return [p[0] for p in self._patterns]

    def _plain_confidence(self, text: str) -> float:
        t = unicodedata_fold(text)
        miss = 1.0
        for _, w, rx in self._patterns:
            if rx.search(t):
                miss *= 1.0 - w
        return 1.0 - miss

    def confidence(self, text: str, decode: bool = True) -> float:
        c = self._plain_confidence(text)
        if decode:
            for _, payload in decode_layers(text):
                c = max(c, self._plain_confidence(payload))
        return c

    def detect(self, text: str, decode: bool = True) -> bool:
        return self.confidence(text, decode) >= self.threshold

    def scan_many(self, texts: Sequence[str]) -> List[bool]:
        return [self.detect(t) for t in texts]


def unicodedata_fold(text: str) -> str:
    """NFKC-normalised text with zero-width and bidi control characters removed, so that look-alike spellings and
    invisible separators do not hide a phrase."""
    import unicodedata
    t = unicodedata.normalize("NFKC", text)
    return "".join(ch for ch in t if unicodedata.category(ch) != "Cf")


def scan_encoded(text: str, detector: Optional[JailbreakDetector] = None, max_depth: int = 4) -> List[Tuple[str, str]]:
    """The decoded payloads of ``text`` that the jailbreak detector flags, as (encoding chain, payload)."""
    det = detector or JailbreakDetector()
    return [(c, p) for c, p in decode_layers(text, max_depth) if det.detect(p, decode=False)]


# ------------------------------------------------------------------------------------------------ prompt policy
@dataclass
class PolicyRule:
    kind: str          # "deny" | "allow" | "require" | "max_length"
    pattern: str
    regex: Optional[re.Pattern] = None


class PromptPolicy:
    """Ordered rule list. Rule text: ``deny:<regex>``, ``allow:<regex>`` (a matching allow rule ends the check with a
    pass), ``require:<regex>`` (every prompt must match), ``max_length:<n>``. ``enforce`` returns (ok, reason)."""

    def __init__(self, rules: Iterable[str] = (), capacity: int = 256):
        self.capacity, self.rules = capacity, []
        for r in rules:
            self.add(r)

    def add(self, rule: str) -> int:
        if len(self.rules) >= self.capacity:
            raise OverflowError("policy is full")
        kind, _, pat = rule.partition(":")
        kind = kind.strip().lower()
        if kind not in ("deny", "allow", "require", "max_length") or not pat:
            raise ValueError(f"bad policy rule {rule!r}")
        if kind == "max_length":
            int(pat)
        self.rules.append(PolicyRule(kind, pat, None if kind == "max_length" else re.compile(pat, re.IGNORECASE)))
        return len(self.rules) - 1

    def add_batch(self, rules: Iterable[str]) -> int:
        return sum(1 for r in rules if self.add(r) >= 0)

    def remove(self, index: int) -> bool:
        if not 0 <= index < len(self.rules):
            return False
        del self.rules[index]
        return True

    def clear(self) -> None:
        self.rules = []

    def policies(self) -> List[str]:
        return [f"{r.kind}:{r.pattern}" for r in self.rules]

    def enforce(self, prompt: str) -> Tuple[bool, str]:
        text = unicodedata_fold(prompt)
        for r in self.rules:
            if r.kind == "max_length":
                if len(text) > int(r.pattern):
                    return False, f"longer than {r.pattern} characters"
            elif r.kind == "allow":
                if r.regex.search(text):
                    break
            elif r.kind == "deny":
                if r.regex.search(text):
                    return False, f"matches deny rule {r.pattern!r}"
        for r in self.rules:
            if r.kind == "require" and not r.regex.search(text):
                return False, f"does not match required {r.pattern!r}"
        return True, ""


# ------------------------------------------------------------------------------------------------ token statistics
def token_anomaly_score(token_probs: Sequence[float]) -> float:
    """Mean negative log-probability (nats per token) of the tokens under the model that produced them."""
    if len(token_probs) == 0:
        return 0.0
    p = torch.as_tensor(token_probs, dtype=torch.float64).clamp(1e-10, 1.0)
    return float(-p.log().mean())


def perplexity(token_probs: Sequence[float]) -> float:
    return math.exp(token_anomaly_score(token_probs))


class TokenAnomalyMonitor:
    """Running record of per-response anomaly scores: a histogram for dashboards and a z-score style warning for a
    response whose score is far above what has been seen."""

    def __init__(self, bins: int = 16, max_score: float = 16.0, warn_sigma: float = 3.0, warmup: int = 20):
        self.bins, self.max_score, self.warn_sigma, self.warmup = bins, max_score, warn_sigma, warmup
        self.counts = [0] * bins
        self.n, self.mean, self.m2 = 0, 0.0, 0.0

    def record(self, score: float) -> bool:
        """Adds the score; True when it is a warning (judged against the scores before it)."""
        warn = self.check_warning(score)
        self.counts[min(self.bins - 1, max(0, int(score / self.max_score * self.bins)))] += 1
        self.n += 1
        d = score - self.mean
        self.mean += d / self.n
        self.m2 += d * (score - self.mean)
        return warn

    def check_warning(self, score: float) -> bool:
        if self.n < self.warmup:
            return False
        sd = math.sqrt(self.m2 / max(1, self.n - 1))
        return score > self.mean + self.warn_sigma * max(sd, 1e-6)

    def histogram(self) -> List[float]:
        total = max(1, sum(self.counts))
        return [c / total for c in self.counts]


# ------------------------------------------------------------------------------------------------ generated text
_SENSITIVE = {
    "private_key": r"-----BEGIN (?:RSA |EC |OPENSSH |DSA )?PRIVATE KEY-----",
    "aws_access_key": r"\bAKIA[0-9A-Z]{16}\b",
    "api_token": r"\b(?:sk|pk|ghp|gho|xox[baprs])[-_][A-Za-z0-9_-]{20,}\b",
    "password_assignment": r"(?i)\b(?:password|passwd|secret|api[_-]?key)\s*[:=]\s*\S{6,}",
    "credit_card": r"\b(?:\d[ -]?){13,19}\b",
    "ssn": r"\b\d{3}-\d{2}-\d{4}\b",
    "email": r"\b[A-Za-z0-9._%+-]+@[A-Za-z0-9.-]+\.[A-Za-z]{2,}\b",
}


def _luhn(digits: str) -> bool:
    s, alt = 0, False
    for ch in reversed(digits):
        d = int(ch)
        if alt:
            d = d * 2 - 9 if d > 4 else d * 2
        s, alt = s + d, not alt
    return s % 10 == 0


class DataExtractionGuard:
    """Finds secrets and personal data in generated text (built-in categories plus caller rules) and redacts them.
    Card numbers count only when they pass the Luhn check."""

    def __init__(self, categories: Optional[Iterable[str]] = None):
        names = list(_SENSITIVE) if categories is None else list(categories)
        self._rules: Dict[str, re.Pattern] = {n: re.compile(_SENSITIVE[n]) for n in names}

    def add_rule(self, name: str, pattern: str) -> None:
        self._rules[name] = re.compile(pattern)

    def remove_rule(self, name: str) -> bool:
        return self._rules.pop(name, None) is not None

    def rules(self) -> List[str]:
        return list(self._rules)

    def findings(self, text: str) -> List[Tuple[str, int, int]]:
        out = []
        for name, rx in self._rules.items():
            for m in rx.finditer(text):
                if name == "credit_card":
                    digits = re.sub(r"\D", "", m.group(0))
                    if not (13 <= len(digits) <= 19 and _luhn(digits)):
                        continue
                out.append((name, m.start(), m.end()))
        return sorted(out, key=lambda f: (f[1], -f[2]))

    def contains_sensitive(self, text: str) -> bool:
        return bool(self.findings(text))

    def redact(self, text: str) -> str:
        out, pos = [], 0
        for name, a, b in self.findings(text):
            if a < pos:
                continue
            out.append(text[pos:a] + f"[{name.upper()}]")
            pos = b
        return "".join(out) + text[pos:]


def _ngrams(text: str, n: int) -> List[Tuple[str, ...]]:
    w = re.findall(r"[a-z0-9]+", text.lower())
    return [tuple(w[i:i + n]) for i in range(len(w) - n + 1)]


def factuality_score(statement: str, reference: str) -> float:
    """Share of the statement's word uni- and bigrams that the reference text also has (bigrams weigh double):
    0 = nothing in the statement is backed by the reference, 1 = every piece of it is."""
    s1, s2 = _ngrams(statement, 1), _ngrams(statement, 2)
    if not s1:
        return 0.0
    r1, r2 = set(_ngrams(reference, 1)), set(_ngrams(reference, 2))
    hit = sum(g in r1 for g in s1) + 2.0 * sum(g in r2 for g in s2)
    return hit / (len(s1) + 2.0 * len(s2))


def factuality_check(statement: str, reference: str, threshold: float = 0.5) -> bool:
    return factuality_score(statement, reference) >= threshold


# ------------------------------------------------------------------------------------------------ training text
_SANITIZERS = {
    "email": (re.compile(r"\b[A-Za-z0-9._%+-]+@[A-Za-z0-9.-]+\.[A-Za-z]{2,}\b"), "[EMAIL]"),
    "url": (re.compile(r"\bhttps?://[^\s<>\"']+"), "[URL]"),
    "ip": (re.compile(r"\b(?:(?:25[0-5]|2[0-4]\d|1?\d?\d)\.){3}(?:25[0-5]|2[0-4]\d|1?\d?\d)\b"), "[IP]"),
    "ssn": (re.compile(r"\b\d{3}-\d{2}-\d{4}\b"), "[SSN]"),
    "phone": (re.compile(r"(?<![\w.])(?:\+?\d{1,3}[ .-]?)?(?:\(\d{2,4}\)|\d{2,4})[ .-]\d{3,4}[ .-]\d{3,4}(?!\w)"), "[PHONE]"),
}


def sanitize_training_text(text: str, kinds: Optional[Iterable[str]] = None) -> Tuple[str, Dict[str, int]]:
    """Replaces e-mail addresses, URLs, IPv4 addresses, national-id numbers and phone numbers with placeholders, in
    that order (so that a URL's host is not first taken for an IP). Returns (clean text, count per kind)."""
    counts: Dict[str, int] = {}
    for k in (_SANITIZERS if kinds is None else kinds):
        rx, repl = _SANITIZERS[k]
        text, counts[k] = rx.subn(repl, text)
    return text, counts


def sanitize_training_batch(texts: Sequence[str], kinds: Optional[Iterable[str]] = None) -> List[str]:
    kinds = None if kinds is None else list(kinds)
    return [sanitize_training_text(t, kinds)[0] for t in texts]


# ------------------------------------------------------------------------------------------------ privacy
class ModelInversionDefense:
    """Makes released gradients (federated updates, gradient APIs) poor material for reconstructing training
    inputs: the update is clipped to ``clip_norm`` in L2 and Gaussian noise of ``noise_scale * clip_norm`` per
    coordinate is added. ``apply`` works in place on one tensor or a list of tensors (one joint norm)."""

    def __init__(self, noise_scale: float = 0.01, clip_norm: float = 1.0, seed: Optional[int] = None):
        self.noise_scale, self.clip_norm = float(noise_scale), float(clip_norm)
        self._gen = None if seed is None else torch.Generator().manual_seed(seed)
        self.applied = 0

    def set_noise(self, scale: float) -> None:
        if scale < 0:
            raise ValueError("noise scale must be non-negative")
        self.noise_scale = float(scale)

    def set_clip(self, norm: float) -> None:
        if norm <= 0:
            raise ValueError("clip norm must be positive")
        self.clip_norm = float(norm)

    def config(self) -> Tuple[float, float]:
        return self.noise_scale, self.clip_norm

    @torch.no_grad()
    def apply(self, grads):
        ts = [grads] if isinstance(grads, torch.Tensor) else list(grads)
        total = torch.sqrt(sum(g.float().pow(2).sum() for g in ts))
        coef = min(1.0, self.clip_norm / (float(total) + 1e-12))
        for g in ts:
            g.mul_(coef)
            if self.noise_scale > 0:
                noise = torch.randn(g.shape, generator=self._gen, dtype=torch.float32) * (self.noise_scale * self.clip_norm)
                g.add_(noise.to(g.device, g.dtype))
        self.applied += 1
        return grads


def membership_inference_defense(logits: torch.Tensor, epsilon: float = 4.0, generator: Optional[torch.Generator] = None,
                                 top1_preserving: bool = True) -> torch.Tensor:
    """Released logits carry less about whether an input was a training member: values are centred and clamped to
    [-epsilon, epsilon] (over-confident members look like everyone else) and Laplace(1 / epsilon) noise is added.
    With ``top1_preserving`` the arg-max class of each row is restored if noise moved it."""
    if epsilon <= 0:
        raise ValueError("epsilon must be positive")
    x = logits.float()
    x = (x - x.mean(-1, keepdim=True)).clamp(-epsilon, epsilon)
    u = torch.rand(x.shape, generator=generator).to(x.device) - 0.5
    noisy = x - (1.0 / epsilon) * u.sign() * torch.log1p(-2.0 * u.abs())
    if top1_preserving:
        top = x.argmax(-1, keepdim=True)
        peak = noisy.amax(-1, keepdim=True)
        noisy = noisy.scatter(-1, top, torch.maximum(noisy.gather(-1, top), peak + 1e-3))
    return noisy.to(logits.dtype)


@torch.no_grad()
def adversarial_smooth(fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, sigma: float = 0.1, samples: int = 16,
                       generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Randomised smoothing: the mean of ``fn`` over ``samples`` Gaussian perturbations of ``x`` (for a classifier's
    probabilities, the smoothed classifier whose prediction is certifiably stable in an L2 ball that grows with sigma)."""
    acc = None
    for _ in range(samples):
        y = fn(x + sigma * torch.randn(x.shape, generator=generator).to(x.device, x.dtype))
        acc = y.float() if acc is None else acc + y.float()
    return acc / samples


def certified_radius(p_top: float, sigma: float) -> float:
    """L2 radius inside which the smoothed classifier's top class cannot change, given a lower bound ``p_top`` on the
    top class probability under noise (Cohen et al. 2019): sigma * Phi^-1(p_top); 0 when p_top <= 1/2."""
    if p_top <= 0.5:
        return 0.0
    p = min(p_top, 1.0 - 1e-12)
    return sigma * float(torch.distributions.Normal(0.0, 1.0).icdf(torch.tensor(p, dtype=torch.float64)))


# ------------------------------------------------------------------------------------------------ fairness
@dataclass
class BiasMetrics:
    """Group fairness of binary decisions between the group with ``sensitive == 1`` and the rest.

    demographic_parity: P(yhat=1 | s=1) - P(yhat=1 | s=0); disparate_impact: the ratio of the smaller of those two
    rates to the larger (the "80 % rule" compares it with 0.8); equalized_odds: the larger of the absolute gaps in
    true-positive rate and false-positive rate (needs labels)."""

    demographic_parity: float = 0.0
    disparate_impact: float = 1.0
    equalized_odds: Optional[float] = None
    tpr_gap: Optional[float] = None
    fpr_gap: Optional[float] = None
    n: int = 0
    threshold: float = 0.5

    @classmethod
    def measure(cls, predictions, sensitive, labels=None, threshold: float = 0.5) -> "BiasMetrics":
        p = torch.as_tensor(predictions, dtype=torch.float64)
        s = torch.as_tensor(sensitive).bool()
        if p.numel() == 0 or p.shape != s.shape:
            raise ValueError("predictions and sensitive attribute must be non-empty and of one shape")
        yhat = p >= threshold

        def rate(mask):
            return float(yhat[mask].double().mean()) if bool(mask.any()) else 0.0

        r1, r0 = rate(s), rate(~s)
        di = 1.0 if max(r1, r0) == 0 else min(r1, r0) / max(r1, r0)
        out = cls(r1 - r0, di, n=int(p.numel()), threshold=threshold)
        if labels is not None:
            y = torch.as_tensor(labels).bool()
            out.tpr_gap = rate(s & y) - rate(~s & y)
            out.fpr_gap = rate(s & ~y) - rate(~s & ~y)
            out.equalized_odds = max(abs(out.tpr_gap), abs(out.fpr_gap))
        return out

    def passes(self, parity_tolerance: float = 0.1, impact_floor: float = 0.8, odds_tolerance: float = 0.1) -> bool:
        ok = abs(self.demographic_parity) <= parity_tolerance and self.disparate_impact >= impact_floor
        return ok and (self.equalized_odds is None or self.equalized_odds <= odds_tolerance)

    def report(self) -> str:
        lines = [f"samples: {self.n} (decision threshold {self.threshold})",
                 f"demographic parity difference: {self.demographic_parity:+.4f}",
                 f"disparate impact ratio: {self.disparate_impact:.4f}"]
        if self.equalized_odds is not None:
            lines.append(f"equalized odds gap: {self.equalized_odds:.4f} (TPR {self.tpr_gap:+.4f}, FPR {self.fpr_gap:+.4f})")
        lines.append("verdict: " + ("within tolerance" if self.passes() else "outside tolerance"))
        return "\n".join(lines)
