"""Published routing-quality results of the reference, kept as data.

Model: 13.14 B total / 1.33 B active parameters; four routing modes x four seeds; hold-out
validation loss as paired differences against unconstrained top-k, with 90 % intervals, read out at
20 k and 30 k steps.  Values transcribed from the reference's figure script
(``tools/gen_figures.py:64-225``) and result pages (``README.md:122-126``,
``docs/06-troute-results.md``); nothing here is measured by this package.
"""

MODES = ("group_limited", "quota_only", "full")

# extra loss in nats: (mean, low, high) of the 90 % interval
LOSS_COST = {
    "20k": {"group_limited": (0.00276, 0.00223, 0.00329), "quota_only": (0.00895, 0.00726, 0.01064),
            "full": (0.00339, 0.00224, 0.00455)},
    "30k": {"group_limited": (0.00192, 0.00114, 0.00270), "quota_only": (0.00895, 0.00751, 0.01039),
            "full": (0.00372, 0.00300, 0.00444)},
}
# the same differences per seed
PER_SEED = {
    "20k": {"group_limited": [0.002659, 0.002195, 0.002931, 0.003251],
            "quota_only": [0.009686, 0.008026, 0.007498, 0.010593],
            "full": [0.003032, 0.003252, 0.002501, 0.004791]},
    "30k": {"group_limited": [0.001513, 0.002640, 0.001219, 0.002305],
            "quota_only": [0.010748, 0.008523, 0.007984, 0.008553],
            "full": [0.003432, 0.003636, 0.003208, 0.004601]},
}
# downstream accuracy difference of `full` against top-k in percentage points (mean, low, high);
# prespecified equivalence bounds +-1.0
DOWNSTREAM_PP = {"HellaSwag acc_norm": (0.158, -0.095, 0.411), "LAMBADA accuracy": (-0.084, -0.406, 0.238)}
EQUIVALENCE_PP = 1.0
# downstream swing at 10 k / 20 k / 30 k steps, percentage points
SWING_STEPS = (10, 20, 30)
SWING_PP = {"group_limited": [0.369, -0.097, -0.645], "full": [0.752, -0.427, -0.577],
            "quota_only": [0.398, 0.058, -1.586]}
# load axis: difference in load entropy and in the coefficient of variation (mean, half-width)
LOAD_ENTROPY = {"group_limited": (0.00018, 0.00033), "quota_only": (0.00035, 0.00026),
                "full": (0.00026, 0.00040)}
LOAD_CV = {"group_limited": (-0.0061, 0.0125), "quota_only": (-0.0137, 0.0094),
           "full": (-0.0094, 0.0147)}
# step-time effect of the routing constraint alone, G = t(top-k) / t(T-Route), two runs
STEP_G = (0.9882, 1.0070)
# small-scale forerunner (2 x 2 factorisation): (mode, hold-out loss, half-width, load entropy)
FORERUNNER = [("global_topk", 6.0302, 0.0003, 0.924), ("quota_only", 6.0313, 0.0002, 0.907),
              ("group_limited", 6.0305, 0.0011, 0.930), ("full", 6.0306, 0.0002, 0.946)]


def conjunction_cost_share(readout: str = "20k") -> float:
    """Loss cost of both constraints together as a share of the quota constraint alone."""
    return LOSS_COST[readout]["full"][0] / LOSS_COST[readout]["quota_only"][0]
