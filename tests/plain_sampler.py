"""A plain restatement of the reference's sampler, for the tests to hold the native host
sampler (and through it the device kernels) to.  Rests on the formulas of
crates/vipera-sampler/src/lib.rs and rng.rs (cited per function); shares no code with the
package under test."""
import math
import struct

MASK = (1 << 64) - 1


def f32(value):
    """Round a Python float to 32-bit, as the reference's `f32` arithmetic does."""
    return struct.unpack("f", struct.pack("f", value))[0]


class Rng:
    """xorshift64* seeded through SplitMix64 (crates/vipera-sampler/src/rng.rs:13-57)."""

    def __init__(self, seed):
        state = ((seed ^ 0x9E3779B97F4A7C15) + 0x9E3779B97F4A7C15) & MASK
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
        self.state = z ^ (z >> 31)

    def next_u64(self):
        x = self.state
        x ^= x >> 12
        x = (x ^ (x << 25)) & MASK
        x ^= x >> 27
        self.state = x
        return (x * 0x2545F4914F6CDD1D) & MASK

    def next_f64(self):
        return (self.next_u64() >> 11) / float(1 << 53)


def penalised(logits, recent, repetition=1.0, presence=0.0, frequency=0.0, bias=()):
    """lib.rs:596-616: for ids seen in `recent`, logit > 0 ? logit / f : logit * f, minus
    presence + frequency * count; then the id's bias."""
    counts = {}
    for token in recent:
        counts[token] = counts.get(token, 0) + 1
    out = list(logits)
    for token, count in counts.items():
        value = out[token]
        if repetition != 1.0:
            value = f32(value / repetition) if value > 0 else f32(value * repetition)
        out[token] = f32(value - f32(presence + f32(frequency * count)))
    for token, value in bias:
        out[token] = f32(out[token] + value)
    return out


def greedy(logits):
    """lib.rs:135-156: the best finite logit, ties to the lowest id."""
    best = None
    for token, value in enumerate(logits):
        if not math.isfinite(value):
            continue
        if best is None or value > logits[best]:
            best = token
    if best is None:
        raise ValueError("no finite logits")
    return best


def temperature(logits, temperature, top_k, top_p, min_p, uniform):
    """lib.rs:172-247, with the head bound of 4096 when top_k is 0 (lib.rs:437)."""
    scale = f32(1.0 / temperature)
    finite = [(token, value) for token, value in enumerate(logits) if math.isfinite(value)]
    ranked = sorted(finite, key=lambda item: (-item[1], item[0]))
    bound = 4096 if top_k == 0 else top_k
    head = ranked[:bound]
    peak = f32(head[0][1] * scale)
    total = 0.0
    for _, value in finite:                                  # every finite logit, in id order
        total = f32(total + f32(math.exp(f32(f32(value * scale) - peak))))

    def weights_of(candidates):
        return [(token, f32(math.exp(f32(f32(value * scale) - peak)))) for token, value in candidates]

    def cut_of(weights):
        target, cumulative = f32(top_p * total), 0.0
        for index, (_, weight) in enumerate(weights):
            cumulative = f32(cumulative + weight)
            if cumulative >= target:
                return index + 1
        return None

    weights = weights_of(head)
    cut = cut_of(weights)
    if top_k == 0 and cut is None and len(head) < len(finite):
        weights = weights_of(ranked)
        cut = cut_of(weights)
    if cut is not None:
        weights = weights[:cut]
    floor = f32(min_p * weights[0][1])
    weights = [item for item in weights if item[1] >= floor]
    mass = 0.0
    for _, weight in weights:
        mass = f32(mass + weight)
    target, running = uniform * mass, 0.0
    for token, weight in weights:
        running += weight
        if target < running:
            return token
    return weights[-1][0]


def logprobs(logits, token, temperature=0.0, top_n=0):
    """lib.rs:302-378: over every finite logit, x = logit / temperature (1 for greedy),
    logprob = x - max - ln(sum exp(x - max)); the token's, and the top_n ids with theirs, best
    first, ties to the lowest id.  (Penalties, where a request has them, are applied to the logits
    first, as in `penalised`.)"""
    t = temperature if temperature > 0.0 else 1.0
    scaled = [(i, f32(v / t)) for i, v in enumerate(logits) if math.isfinite(v)]
    peak = max(x for _, x in scaled)
    mass = 0.0
    for _, x in scaled:
        mass = f32(mass + f32(math.exp(f32(x - peak))))
    log_mass = f32(math.log(mass))
    of = lambda x: f32(f32(x - peak) - log_mass)  # noqa: E731
    chosen = of(f32(logits[token] / t))
    top = sorted(scaled, key=lambda item: (-item[1], item[0]))[:top_n]
    return chosen, [(i, of(x)) for i, x in top]
