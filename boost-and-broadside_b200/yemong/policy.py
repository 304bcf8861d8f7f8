"""The rollout step of the policy on CUDA kernels end to end, mirroring ``YemongPolicy`` of the
reference (models/yemong/policy.py:135-373).

``YemongPolicy`` here has the reference's constructor arguments, sub-module names and parameter
names (``encoder``, ``bullet_encoder``, ``yemong_layers``, ``action_head``, ``value_head_local``,
``team_pma``, ``value_head_win``, ``next_state_head``), so a reference ``state_dict`` loads
unchanged.  ``get_action_and_value`` (policy.py:291-373) runs, from the coordinators' raw feature
vectors on: the encoder kernels, the trunk in one call on the packed state, the head kernels,
TeamPMA and the action draw.  The ``FeatureCoordinator`` objects are the caller's and run as they
are.  ``evaluate_actions`` (policy.py:379-516) is mirrored as a forward: evaluation, crossover and
logging call it without gradients.  For the PPO update itself -- ``evaluate_actions`` differentiated
-- keep the reference's policy and swap its blocks for this package's ``YemongBlock``: the trunk then
runs forward and backward here, and the reference's encoders and heads, which have no backward in
this package, stay torch modules.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .encoder import BulletEncoder, ShipEncoder
from .griffin import YemongBlock
from .heads import HeadMLP, NextStateHead, TeamPMA, evaluate_action, sample_action
from .trunk import YemongTrunk

TOTAL_ACTION_LOGITS = 12  # constants.py:43


class YemongPolicy(YemongTrunk):
    """Encoder -> n x YemongBlock -> heads (policy.py:135-214), rollout path."""

    def __init__(self, model_config, coordinator, num_value_components: int, num_ships: int,
                 team_pma_k: tuple[int, ...], bullet_coordinator=None) -> None:
        nn.Module.__init__(self)   # sub-modules are registered below in the reference's order
        D = model_config.d_model
        self.d_model = self._d_model = D
        self.n_heads = model_config.n_heads
        self.n_temporal = self._n_temporal = model_config.n_temporal_per_block
        self._K = num_value_components
        self._num_ships = num_ships
        self._team_pma_k = tuple(team_pma_k)
        self.coordinator = coordinator
        self.encoder = ShipEncoder(model_config, coordinator, num_ships=num_ships)
        self.bullet_encoder = (BulletEncoder(model_config, bullet_coordinator)
                               if model_config.reads_bullets and bullet_coordinator is not None else None)
        self.yemong_layers = nn.ModuleList([YemongBlock(model_config) for _ in range(model_config.n_yemong_blocks)])
        self.action_head = HeadMLP(D, TOTAL_ACTION_LOGITS)
        self.value_head_local = HeadMLP(D, num_value_components)
        if self._team_pma_k:
            self.team_pma = TeamPMA(D, model_config.n_heads)
            self.value_head_win = HeadMLP(D, len(self._team_pma_k))
        self.next_state_head = NextStateHead(D, coordinator.total_prediction_dimension)

    @property
    def num_recurrent_tokens(self) -> int:
        return self._num_ships

    def _encode_bullets(self, obs):
        if self.bullet_encoder is None or obs.bullets is None:
            return None, None
        active = next(v for k, v in obs.bullets.items() if getattr(k, "name", str(k)).upper().endswith("ACTIVE"))
        return self.bullet_encoder(obs), active

    @torch.no_grad()
    def get_action_and_value(self, obs, hidden: torch.Tensor, generator: torch.Generator | None = None):
        """One rollout step (policy.py:291-373): returns (action (B, N, 3), logprob (B, N),
        value (B, N, K), pred_next (B, N, pred_dim), new_hidden)."""
        alive = obs["alive"]
        x = self.encoder(obs)
        bullets, bullet_mask = self._encode_bullets(obs)
        x, new_hidden = self.step(x, alive, hidden, bullets=bullets, bullet_mask=bullet_mask)
        N = self._num_ships
        x_ships = x[:, :N, :].contiguous()
        logits = self.action_head(x_ships)
        pred_next = self.next_state_head(x_ships)
        value = self.value_head_local(x_ships)
        if self._team_pma_k:
            x_team = self.team_pma(x_ships, obs["team_id"][:, :N], alive[:, :N])
            win_val = self.value_head_win(x_team)
            for i, k in enumerate(self._team_pma_k):
                value[:, :, k] = win_val[:, :, i]
        action, logprob = sample_action(logits, generator)
        return action, logprob, value, pred_next, new_hidden

    @torch.no_grad()
    def evaluate_actions(self, obs, actions: torch.Tensor, initial_hidden: torch.Tensor, alive_mask: torch.Tensor,
                         done_mask: torch.Tensor | None = None, return_encoder_output: bool = False):
        """The rollout re-evaluated over T steps (policy.py:379-516), without gradients: obs with
        (T, B, N+M, ...) tensors, actions (T, B, N, 3).  Returns (logprob (T, B, N), entropy (T, B, N),
        value (T, B, N, K), logits (T, B, N, 12), encoder output or None, pred_next (T, B, N, pred_dim))."""
        T, B, N = actions.shape[:3]
        flat = type(obs)(
            data={k: v.reshape(T * B, *v.shape[2:]) for k, v in obs.items()},
            bullets=None if obs.bullets is None else {k: v.reshape(T * B, *v.shape[2:]) for k, v in obs.bullets.items()},
        )
        x = self.encoder(flat)
        NM, D = x.shape[1], x.shape[2]
        x = x.reshape(T, B, NM, D)
        bullets, bullet_mask = self._encode_bullets(flat)
        z = x if return_encoder_output else None
        x, _ = self.sequence(x, alive_mask, initial_hidden, done_mask, bullets=bullets, bullet_mask=bullet_mask)
        x_ships = x[:, :, :N, :].contiguous()
        logits = self.action_head(x_ships)
        pred_next = self.next_state_head(x_ships)
        value = self.value_head_local(x_ships)
        if self._team_pma_k:
            pooled = self.team_pma(x_ships.reshape(T * B, N, D), obs["team_id"][:, :, :N].reshape(T * B, N),
                                   alive_mask[:, :, :N].reshape(T * B, N))
            win_val = self.value_head_win(pooled.reshape(T, B, N, D))
            for i, k in enumerate(self._team_pma_k):
                value[..., k] = win_val[..., i]
        logprob, entropy = evaluate_action(logits, actions)
        return logprob, entropy, value, logits, z, pred_next
