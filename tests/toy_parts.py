"""Toy parts and toy architectures for the tests: a mixer with state of its own, another
position encoding, a feed-forward that routes every token to one of several experts, an
architecture that mixes both kinds of layer, one whose execution order names a layer
twice and lets a layer read another layer's cache, and two other arrangements of a layer (four
norms around the two sub-layers; mixer and feed-forward side by side under one norm) in a model
that also scales its embedding rows.  They are defined and
registered here, outside the package; ``register()`` is called by the tests, and by a process
that lists this file in VIPERA_PLUGINS (bin/trace_run in the replay tests)."""
import torch


def register():
    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200 import parts  # noqa: F401
    from vipera_rs_b200.config import (ARCHITECTURES, BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LayerSpec,
                                       ModelSpec, PartSpec, Qwen2Config, ScheduleEntry, qwen2_model_spec,
                                       register_architecture)
    from vipera_rs_b200.parts import Block, FeedForward, FixedState, Mixer, NormedInput, PositionEncoding
    from vipera_rs_b200.weights import TensorSpec

    if "toy_running_mean" in MIXERS:
        return

    class RunningMean(Mixer):
        """A mixer with state of its own: out_t = W . mean(h_0 .. h_t).  It keeps, per request,
        the running sum of h and the count: one float32 row of hidden + 1 numbers, whatever
        the length.  Written with torch operations; it talks to the host, so it is not captured."""

        graph_safe = False

        @classmethod
        def schema(cls, params, prefix):
            return {f"{prefix}.mix.weight": TensorSpec((params["hidden_size"], params["hidden_size"]))}

        def __init__(self, params, prefix, tensors, dtype, device):
            super().__init__(params, prefix, tensors, dtype, device)
            self.hidden = params["hidden_size"]
            self.weight = tensors[f"{prefix}.mix.weight"].to(device=device, dtype=torch.float32)

        @classmethod
        def cache_request_for(cls, params):
            return FixedState((params["hidden_size"] + 1,), torch.float32)

        def forward(self, ctx, h, residual, cache, writes_cache):
            slots, fresh = ctx.state_slots.tolist(), ctx.fresh.tolist()
            offset = 0
            for entry, count in enumerate(ctx.host_counts):
                state = cache.data[slots[entry]]
                if fresh[entry]:
                    state.zero_()
                rows = h[offset:offset + count].float()
                sums = state[: self.hidden] + torch.cumsum(rows, dim=0)
                counts = state[self.hidden] + torch.arange(1, count + 1, device=h.device, dtype=torch.float32)
                residual[offset:offset + count] += (sums / counts[:, None]) @ self.weight.T
                state[: self.hidden] = sums[-1]
                state[self.hidden] = counts[-1]
                offset += count

    class LearnedShift(PositionEncoding):
        """Another position encoding: a learned vector per position added to q and k.  The fused
        kernels do not know it (style None), so the attention part calls apply()."""

        style = None

        @classmethod
        def schema(cls, params, prefix):
            return {f"{prefix}.shift.weight": TensorSpec((params["max_positions"], params["head_dim"]))}

        def __init__(self, params, prefix, tensors, dtype, device):
            super().__init__(params, prefix, tensors, dtype, device)
            self.table = tensors[f"{prefix}.shift.weight"].to(device=device, dtype=torch.float32)

        def apply(self, ctx, q, k):
            shift = self.table[ctx.positions.long()][:, None, :]
            q += shift
            k += shift

    class RoutedExperts(FeedForward):
        """A feed-forward with routing: every token goes to the expert whose router row scores
        it highest (the lowest index wins a tie), and the expert is ``down(relu(up(h)))``.
        Written with torch operations that stay on the device (every expert is computed and the
        others are masked out), so it can be captured in a graph."""

        @classmethod
        def schema(cls, params, prefix):
            hidden, inter, experts = params["hidden_size"], params["expert_size"], params["experts"]
            schema = {f"{prefix}.router.weight": TensorSpec((experts, hidden), store="float32")}
            for e in range(experts):
                schema[f"{prefix}.experts.{e}.up.weight"] = TensorSpec((inter, hidden))
                schema[f"{prefix}.experts.{e}.down.weight"] = TensorSpec((hidden, inter))
            return schema

        def __init__(self, params, prefix, tensors, dtype, device):
            super().__init__(params, prefix, tensors, dtype, device)
            self.experts = params["experts"]
            to = lambda name: tensors[f"{prefix}.{name}"].to(device=device, dtype=torch.float32)  # noqa: E731
            self.router = to("router.weight")
            self.up = torch.stack([to(f"experts.{e}.up.weight") for e in range(self.experts)])
            self.down = torch.stack([to(f"experts.{e}.down.weight") for e in range(self.experts)])

        def forward(self, ctx, h, residual):
            x = h.float()
            scores = x @ self.router.T                                            # [tokens, experts], 32-bit
            chosen = torch.nn.functional.one_hot(scores.argmax(dim=1), self.experts).to(x.dtype)
            every = torch.einsum("eti,ehi->eth", torch.relu(torch.einsum("th,eih->eti", x, self.up)), self.down)
            residual += torch.einsum("eth,te->th", every, chosen)

    class SandwichBlock(Block):
        """Four norms: ``x += post_norm(mixer(pre_norm(x)))`` and the same around the feed-forward.
        Mixers and feed-forwards add into the stream they are given, so each sub-layer is run on a
        zeroed stream of its own, which the second norm then reads."""

        roles = {"mixer_norm": NORMS, "mixer": MIXERS, "mixer_post_norm": NORMS,
                 "ffn_norm": NORMS, "ffn": FEED_FORWARDS, "ffn_post_norm": NORMS}

        def _sub_layer(self, ctx, residual, norm, run, post_norm):
            branch = torch.zeros_like(residual)
            run(NormedInput(ctx, norm, residual).tensor(), branch)
            out = torch.empty(residual.shape, dtype=ctx.dtype, device=residual.device)
            post_norm.forward(ctx, branch, out)
            residual += out.float() * self.params.get("branch_scale", 1.0)

        def forward(self, ctx, residual, cache, writes_cache):
            self._sub_layer(ctx, residual, self.mixer_norm,
                            lambda h, branch: self.mixer.forward(ctx, h, branch, cache, writes_cache), self.mixer_post_norm)
            self._sub_layer(ctx, residual, self.ffn_norm,
                            lambda h, branch: self.ffn.forward(ctx, h, branch), self.ffn_post_norm)

    class ParallelBlock(Block):
        """One norm; mixer and feed-forward both read it and both add into the stream."""

        roles = {"norm": NORMS, "mixer": MIXERS, "ffn": FEED_FORWARDS}

        def forward(self, ctx, residual, cache, writes_cache):
            h = NormedInput(ctx, self.norm, residual).tensor()
            self.mixer.forward(ctx, h, residual, cache, writes_cache)
            self.ffn.forward(ctx, h, residual)

    BLOCKS.register("toy_sandwich", SandwichBlock)
    BLOCKS.register("toy_parallel", ParallelBlock)
    MIXERS.register("toy_running_mean", RunningMean)
    POSITION_ENCODINGS.register("toy_learned_shift", LearnedShift)
    FEED_FORWARDS.register("toy_routed_experts", RoutedExperts)

    def toy_state_spec(config):
        """Layer 0 mixes with the running mean, layer 1 with attention."""
        base = qwen2_model_spec(config)
        first = base.layers[0]
        toy = first.with_parts(mixer=PartSpec("toy_running_mean", {"hidden_size": config.hidden_size}))
        return ModelSpec(**{**base.__dict__, "layers": [toy] + base.layers[1:], "architecture": "ToyStateLM"})

    def toy_shared_spec(config):
        """Layer 0 runs twice (cache slots 0 and 1), then layer 1 reads slot 0 without writing."""
        base = qwen2_model_spec(config)
        return ModelSpec(**{**base.__dict__, "architecture": "ToySharedLM",
                            "schedule": [ScheduleEntry(0, 0), ScheduleEntry(0, 1), ScheduleEntry(1, 0, False)]})

    def toy_routed_spec(config):
        """Layer 0 feeds forward through routed experts, layer 1 through SwiGLU."""
        base = qwen2_model_spec(config)
        first = base.layers[0]
        routed = first.with_parts(ffn=PartSpec("toy_routed_experts", {"hidden_size": config.hidden_size,
                                                                      "expert_size": 48, "experts": 5}))
        return ModelSpec(**{**base.__dict__, "layers": [routed] + base.layers[1:], "architecture": "ToyRoutedLM"})

    def toy_arranged_spec(config):
        """Layer 0 has four norms, layer 1 runs mixer and feed-forward side by side under one
        norm, and the embedding rows are scaled."""
        base = qwen2_model_spec(config)
        first, second = base.layers[0], base.layers[1]
        norm = first.parts["mixer_norm"]
        sandwich = LayerSpec(block="toy_sandwich", prefix=first.prefix,
                             parts={**first.parts, "mixer_post_norm": norm, "ffn_post_norm": norm},
                             names={**first.names, "mixer_post_norm": "post_mixer_norm", "ffn_post_norm": "post_ffn_norm"},
                             params={"branch_scale": 0.5})
        parallel = LayerSpec(block="toy_parallel", prefix=second.prefix,
                             parts={"norm": norm, "mixer": second.parts["mixer"], "ffn": second.parts["ffn"]},
                             names={"norm": "input_layernorm", "mixer": "self_attn", "ffn": "mlp"})
        return ModelSpec(**{**base.__dict__, "layers": [sandwich, parallel], "architecture": "ToyArrangedLM",
                            "embedding_scale": 3.0})

    register_architecture("ToyArrangedLM", Qwen2Config.from_dict, toy_arranged_spec)
    register_architecture("ToyRoutedLM", Qwen2Config.from_dict, toy_routed_spec)
    register_architecture("ToyStateLM", Qwen2Config.from_dict, toy_state_spec)
    register_architecture("ToySharedLM", Qwen2Config.from_dict, toy_shared_spec)


