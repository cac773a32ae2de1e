"""Reading a tracing build's marks (OMNIA_TIMELINE=1, see csrc/common.cuh and csrc/build.py).

Block 0 of every kernel stamps the GPU's clock when its wait for the kernel before it is over,
that is, when that kernel has finished. The distance between two kernels' stamps is therefore the
time the earlier one takes in the stream as it really runs, launch overlaps included.
"""

from __future__ import annotations

import statistics

from mlx_omnia_b200.csrc import build


def spans() -> list[tuple[str, int, float]]:
    """(library, source line of the kernel's wait, microseconds until the next kernel could start)
    for every kernel launched since the marks were last read, in launch order; the last kernel
    has no successor and is left out. Synchronise the device first."""
    over = [(t, lib, line) for t, lib, line, phase, _, _ in build.timeline() if phase == 1]
    return [(lib, line, (over[i + 1][0] - t) / 1000.0) for i, (t, lib, line) in enumerate(over[:-1])]


def by_layer(kernels: list[tuple[str, int, float]], anchor: str) -> list[str]:
    """The spans of a model step as text: kernels of the repeating part (found by the distance
    between launches of library `anchor`, one per layer) by their place in a layer, with the
    median over layers; the kernels before and after the layers one by one."""
    at = [i for i, (lib, _, _) in enumerate(kernels) if lib == anchor or lib == anchor + "_wide"]
    if len(at) < 2:
        return [f"{lib}:{line} {us:8.2f} us" for lib, line, us in kernels]
    period = at[1] - at[0]
    labels = [kernel[:2] for kernel in kernels]
    first = at[0]  # walk back from the first anchor for as long as a layer later looks the same
    while first > 0 and labels[first - 1] == labels[first - 1 + period]:
        first -= 1
    layers = 1
    while first + (layers + 1) * period <= len(labels) and \
            labels[first + layers * period: first + (layers + 1) * period] == labels[first: first + period]:
        layers += 1
    lines = [f"before the layers   {lib}:{line:<4d} {us:8.2f} us" for lib, line, us in kernels[:first]]
    total = 0.0
    for place in range(period):
        values = [kernels[first + layer * period + place][2] for layer in range(layers)]
        lib, line, _ = kernels[first + place]
        total += statistics.median(values)
        lines.append(f"layer, kernel {place:2d}    {lib}:{line:<4d} {statistics.median(values):8.2f} us "
                     f"(min {min(values):.2f}, max {max(values):.2f}, {layers} layers)")
    lines.append(f"a layer             {total:8.2f} us")
    lines += [f"after the layers    {lib}:{line:<4d} {us:8.2f} us" for lib, line, us in kernels[first + layers * period:]]
    return lines
