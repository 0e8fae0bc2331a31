"""Bag-of-embeddings sentiment classifier: byte-pair tokenizer trained on the corpus, ``Embedding`` + mean pooling +
``Linear``, padded batches from ``BatchCollator``."""
from _common import device, seed  # first: makes the package importable from a checkout
import torch

import SneppX_ALG as sx
from sneppx.nn import Embedding, Linear, Module
from sneppx.optim.zoo import AdamW

GOOD = ["a wonderful and moving film", "great acting and a great story", "i loved every minute", "brilliant, funny, warm",
        "one of the best this year", "a joy to watch", "beautiful and clever", "fantastic cast, superb writing"]
BAD = ["a dull and lifeless film", "terrible acting and a weak story", "i hated every minute", "boring, slow, cold",
       "one of the worst this year", "a chore to watch", "ugly and stupid", "awful cast, lazy writing"]


class BagOfEmbeddings(Module):
    def __init__(self, vocab: int, dim: int = 32, device=None):
        super().__init__()
        self.emb, self.out = Embedding(vocab, dim, device=device), Linear(dim, 2, device=device)

    def forward(self, ids, pad_id=0):
        mask = (ids != pad_id).unsqueeze(-1).float()
        return self.out((self.emb(ids) * mask).sum(1) / mask.sum(1).clamp_min(1.0))


def main(steps: int = 150) -> float:
    seed(3)
    dev = device()
    tok = sx.SimpleTokenizer(300)
    texts, labels = GOOD + BAD, [1] * len(GOOD) + [0] * len(BAD)
    collate = sx.BatchCollator(padding_value=0)
    ids = collate([[t + 1 for t in tok.encode(s)] for s in texts]).to(dev)      # shift by one: 0 is the padding id
    y = torch.tensor(labels, device=dev)
    model = BagOfEmbeddings(302, device=dev)
    opt = AdamW(model.parameters(), lr=2e-2, weight_decay=0.0)
    for _ in range(steps):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(ids), y)
        loss.backward()
        opt.step()
    test = collate([[t + 1 for t in tok.encode(s)] for s in ("a great and moving story", "a weak and boring film")]).to(dev)
    with torch.no_grad():
        acc = (model(ids).argmax(-1) == y).float().mean().item()
        pred = model(test).argmax(-1).tolist()
    print(f"train accuracy {acc:.2f}; held-out predictions (want [1, 0]): {pred}")
    return acc


if __name__ == "__main__":
    main()
