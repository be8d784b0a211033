"""End-to-end training on the CPU with the framework's own nn / optim / data / train layers: the loss must fall well below its initial value
for an MLP, a transformer encoder, a CNN, an LSTM and a VAE (the same five families the reference trains in its integration suite)."""
import pytest
import torch

from ferrotorch_b200 import data, nn, optim


def _fit(model, batches, loss_fn, opt, steps):
    first = last = None
    for i in range(steps):
        x, y = batches[i % len(batches)]
        opt.zero_grad()
        loss = loss_fn(model(x), y)
        loss.backward()
        opt.step()
        first = float(loss) if first is None else first
        last = float(loss)
    return first, last


def test_mlp_classification_with_dataloader():
    torch.manual_seed(0)
    X = torch.randn(256, 20)
    y = (X[:, :3].sum(1) > 0).long()
    loader = data.DataLoader(data.TensorDataset(X, y), batch_size=32, shuffle=True, seed=0)
    model = nn.Sequential(nn.Linear(20, 64), nn.ReLU(), nn.Linear(64, 2))
    opt = optim.AdamW(model.parameters(), lr=1e-2)
    lossf = nn.CrossEntropyLoss()
    first = last = None
    for epoch in range(8):
        for xb, yb in loader:
            opt.zero_grad()
            loss = lossf(model(xb), yb)
            loss.backward()
            opt.step()
            first = float(loss) if first is None else first
            last = float(loss)
    assert last < 0.5 * first
    assert (model(X).argmax(1) == y).float().mean() > 0.9


def test_transformer_encoder_copy_task():
    torch.manual_seed(0)
    V, S, E = 16, 8, 32
    emb, enc, head = nn.Embedding(V, E), nn.TransformerEncoder(nn.TransformerEncoderLayer(E, 4, 64, dropout=0.0, batch_first=True), 2), nn.Linear(E, V)
    model = nn.Sequential(emb, enc, head)
    batches = [(t, t) for t in (torch.randint(0, V, (16, S)) for _ in range(4))]
    first, last = _fit(model, batches, lambda o, y: torch.nn.functional.cross_entropy(o.reshape(-1, V), y.reshape(-1)), optim.Adam(model.parameters(), lr=3e-3), 120)
    assert last < 0.5 * first


def test_cnn_lstm_and_vae():
    torch.manual_seed(0)
    cnn = nn.Sequential(nn.Conv2d(1, 8, 3, padding=1), nn.BatchNorm2d(8), nn.ReLU(), nn.MaxPool2d(2), nn.Flatten(), nn.Linear(8 * 7 * 7, 4))
    xs = torch.randn(64, 1, 14, 14)
    ys = (xs.mean((1, 2, 3)) > 0).long() + 2 * (xs[:, :, :7].mean((1, 2, 3)) > 0).long()
    first, last = _fit(cnn, [(xs, ys)], nn.CrossEntropyLoss(), optim.Sgd(cnn.parameters(), lr=0.1, momentum=0.9), 60)
    assert last < 0.9 * first

    class Seq(nn.Module):
        def __init__(self):
            super().__init__()
            self.rnn, self.out = nn.LSTM(4, 16, batch_first=True), nn.Linear(16, 1)

        def forward(self, x):
            h, _ = self.rnn(x)
            return self.out(h[:, -1]).squeeze(-1)
    seq = Seq()
    x = torch.randn(64, 10, 4)
    y = x[:, :, 0].sum(1)
    first, last = _fit(seq, [(x, y)], nn.MSELoss(), optim.Adam(seq.parameters(), lr=1e-2), 150)
    assert last < 0.5 * first

    class Vae(nn.Module):
        def __init__(self):
            super().__init__()
            self.enc, self.mu, self.lv, self.dec = nn.Linear(20, 32), nn.Linear(32, 4), nn.Linear(32, 4), nn.Sequential(nn.Linear(4, 32), nn.ReLU(), nn.Linear(32, 20))

        def forward(self, x):
            h = torch.relu(self.enc(x))
            mu, lv = self.mu(h), self.lv(h)
            z = mu + torch.randn_like(mu) * (0.5 * lv).exp()
            return self.dec(z), mu, lv
    vae = Vae()
    base = torch.randn(128, 4) @ torch.randn(4, 20)

    def vae_loss(out, target):
        rec, mu, lv = out
        return torch.nn.functional.mse_loss(rec, target) + 1e-3 * (-0.5 * (1 + lv - mu ** 2 - lv.exp()).mean())
    first, last = _fit(vae, [(base, base)], vae_loss, optim.Adam(vae.parameters(), lr=5e-3), 200)
    assert last < 0.5 * first
