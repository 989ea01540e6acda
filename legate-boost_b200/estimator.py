"""A thin boosting-round driver over ``Tree``: just enough of ``LBRegressor`` / ``LBClassifier`` to
grow an ensemble and measure rounds per second.

It restates the reference's round (legateboost/legateboost.py:254-298): gradient of the objective
at the current prediction, times the learning rate (``_get_weighted_gradient``, :189-224, hessian
floored at 1e-8), ``Tree(...).set_random_state(rs).fit(X, g, h)``, ``train_pred += tree.predict(X)``.
Objectives: squared error (objectives.py:119-147) and multi-class / binary log loss
(objectives.py:477-531).  Everything else of the estimators (callbacks, metrics registry, other base
models, update, sklearn plumbing) is outside the tree-building hot path and is not provided.
Arrays are torch CUDA tensors; under ``torch.distributed`` each rank holds a block of rows.
"""
from copy import deepcopy
from typing import List, Optional

import numpy as np
import torch

from . import library as L
from .tree import Sketch, Tree, _row_layout


def _all_sum(t: torch.Tensor) -> torch.Tensor:
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t)
    return t


class _SquaredError:
    code = 0  # LBK_SQUARED_ERROR

    def gradient(self, y, pred):
        return pred - y, torch.ones_like(pred)

    def transform(self, pred):
        return pred

    def init(self, y, average):
        if not average:
            return torch.zeros(y.shape[1], dtype=torch.float64, device=y.device)
        s = _all_sum(torch.cat([y.sum(dim=0), torch.tensor([float(y.shape[0])], dtype=torch.float64, device=y.device)]))
        return s[:-1] / s[-1]

    def metric(self, y, pred):
        s = _all_sum(torch.cat([((y - pred) ** 2).sum(dim=0), torch.tensor([float(y.shape[0])], dtype=torch.float64, device=y.device)]))
        return float((s[:-1] / s[-1]).mean())


class _LogLoss:
    code = 1  # LBK_LOG_LOSS

    def gradient(self, y, pred):
        if pred.shape[1] == 1:
            return pred - y, pred * (1.0 - pred)
        label = y.to(torch.int64).reshape(-1)
        h = pred * (1.0 - pred)
        g = pred.clone()
        g[torch.arange(label.numel(), device=g.device), label] -= 1.0
        return g, h

    def transform(self, pred):
        if pred.shape[1] == 1:
            return 1.0 / (1.0 + torch.exp(-pred))
        s = pred.max(dim=1, keepdim=True).values
        e = torch.exp(pred - s)
        return e / e.sum(dim=1, keepdim=True)

    def init(self, y, average):
        mx = torch.tensor([float(y.max()) if y.numel() else 0.0], dtype=torch.float64, device=y.device)
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        num_class = int(mx.item()) + 1
        n_targets = num_class if num_class > 2 else 1
        if not average:
            return torch.zeros(n_targets, dtype=torch.float64, device=y.device)
        counts = _all_sum(torch.bincount(y.reshape(-1).to(torch.int64), minlength=num_class).to(torch.float64))
        prob = counts / counts.sum()
        if n_targets == 1:
            return -torch.log(1.0 / prob[1:2] - 1.0)
        return torch.log(prob)

    def metric(self, y, pred):
        eps = torch.finfo(pred.dtype).eps
        p = pred.clamp(eps, 1 - eps)
        if p.shape[1] == 1:
            yy = y.reshape(-1)
            p = p.reshape(-1)
            ll = -(yy * torch.log(p) + (1 - yy) * torch.log(1 - p))
        else:
            label = y.to(torch.int64).reshape(-1)
            ll = -torch.log(p[torch.arange(label.numel(), device=p.device), label])
        s = _all_sum(torch.stack([ll.sum(), torch.tensor(float(ll.numel()), dtype=torch.float64, device=p.device)]))
        return float(s[0] / s[1])


class _LBBase:
    _objective = None

    def __init__(self, n_estimators: int = 100, learning_rate: float = 0.1, init: Optional[str] = "average",
                 base_models=(Tree(max_depth=6),), random_state=None, verbose: int = 0, fixed_sketch: bool = False):
        # fixed_sketch (an extension, off by default): the first tree of every base model saves its
        # split proposals and binned matrix, the later ones reuse them instead of sampling and
        # binning X again; the trees then differ from the reference's, which re-samples per tree
        self.fixed_sketch = fixed_sketch
        self.n_estimators = n_estimators
        self.learning_rate = learning_rate
        self.init = init
        self.base_models = base_models
        self.random_state = random_state
        self.verbose = verbose

    def _check(self, X, y):
        if not (torch.is_tensor(X) and X.is_cuda):
            raise ValueError("X must be a CUDA tensor (there is no CPU path)")
        if X.dtype not in (torch.float32, torch.float64):
            X = X.to(torch.float32)  # integer X -> float32 (reference: input_validation.py:73-75)
        y = torch.as_tensor(y, device=X.device).to(torch.float64)  # y -> float64 (:85)
        if y.dim() == 1:
            y = y[:, None]
        if y.shape[0] != X.shape[0]:
            raise ValueError("Number of labels does not match number of samples.")
        return X, y

    def _weighted_gradient(self, y, raw_pred):
        """g * learning_rate and h floored at 1e-8 at the current raw prediction, in one pass over the
        rows (`lbk_gradient`; reference: `_get_weighted_gradient`, legateboost.py:189-224)."""
        code = getattr(self._obj, "code", None)
        if code is None:  # an objective the library has no kernel for
            g, h = self._obj.gradient(y, self._obj.transform(raw_pred))
            return g * self.learning_rate, torch.clamp(h, min=1e-8)
        raw_pred = raw_pred.contiguous()
        y = y.contiguous()
        g = torch.empty_like(raw_pred)
        h = torch.empty_like(raw_pred)
        ctx = L.context(raw_pred.device.index)
        with torch.cuda.device(raw_pred.device):
            ctx.check(ctx.lib.lbk_gradient(ctx.handle, code, raw_pred.data_ptr(), y.data_ptr(), raw_pred.shape[0],
                                           raw_pred.shape[1], float(self.learning_rate), g.data_ptr(), h.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream))
        return g, h

    def fit(self, X, y):
        X, y = self._check(X, y)
        if not isinstance(self.base_models, tuple) or len(self.base_models) == 0:
            raise ValueError("base_models should be a tuple")
        self.n_features_in_ = X.shape[1]
        self.models_: List[Tree] = []
        rs = self.random_state
        self.random_state_ = rs if isinstance(rs, np.random.RandomState) else np.random.RandomState(rs)
        self._obj = self._objective()
        self.model_init_ = self._obj.init(y, self.init == "average")
        self.train_metric_: List[float] = []
        train_pred = self.model_init_.repeat(X.shape[0], 1)
        layout = _row_layout(X.shape[0])  # this rank's block of rows: the same for every tree
        sketches = {}
        for i in range(self.n_estimators):
            g, h = self._weighted_gradient(y, train_pred)
            tree = deepcopy(self.base_models[i % len(self.base_models)]).set_random_state(self.random_state_)
            tree.row_layout = layout
            if self.fixed_sketch:
                tree.sketch = sketches.setdefault(i % len(self.base_models), Sketch())
            tree.fit(X, g, h)
            tree.sketch = None  # the buffer belongs to this fit, not to the tree
            self.models_.append(tree)
            train_pred += tree.predict(X)
            if self.verbose:
                m = self._obj.metric(y, self._obj.transform(train_pred))
                self.train_metric_.append(m)
                print("[%d] train: %.6f" % (i, m))
        self._train_pred = train_pred
        return self

    def predict_raw(self, X):
        if X.shape[1] != self.n_features_in_:
            raise ValueError("X.shape[1] = {} should be equal to {}".format(X.shape[1], self.n_features_in_))
        pred = self.model_init_.repeat(X.shape[0], 1)
        if self.models_:
            pred += Tree.batch_predict(self.models_, X)
        return pred

    def __iter__(self):
        return iter(self.models_)

    def __getitem__(self, i):
        return self.models_[i]

    def __len__(self):
        return len(self.models_)


class LBRegressor(_LBBase):
    """Gradient-boosted regression with the squared-error objective."""

    _objective = _SquaredError

    def predict(self, X):
        pred = self._obj.transform(self.predict_raw(X))
        return pred.squeeze(1) if pred.shape[1] == 1 else pred


class LBClassifier(_LBBase):
    """Gradient-boosted classification with the log-loss objective."""

    _objective = _LogLoss

    def predict_proba(self, X):
        pred = self._obj.transform(self.predict_raw(X))
        if pred.shape[1] == 1:
            pred = torch.cat([1.0 - pred, pred], dim=1)
        return pred

    def predict(self, X):
        return self.predict_proba(X).argmax(dim=1)
