"""CPU checks of bench.py's workload tables: layer lists and algorithmic work of the five configurations."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_workload_layer_lists_and_bit_op_totals():
    import bench

    w = bench.WORKLOADS
    # SC conv layers per model: ResNet-18 has 16 3x3 + 3 1x1 SC convs, ResNet-34 32 + 3, VGG-16 13 + the classifier
    assert sum(l[6] for l in w["resnet18"]["layers"]) == 19
    assert sum(l[6] for l in w["resnet34"]["layers"]) == 35
    assert sum(l[6] for l in w["vgg16"]["layers"]) == 14
    # forward bit-operations per batch, 2 * L * N*OH*OW * Cout * Cin*KH*KW (in units of 10^12)
    tera = {k: bench.bitops_per_image(w[k]["layers"]) * w[k]["batch"] / 1e12 for k in ("resnet18", "resnet34", "conv5x5")}
    assert abs(tera["resnet18"] - 27.78) < 0.01
    assert abs(tera["resnet34"] - 87.13) < 0.01
    assert abs(tera["conv5x5"] - 0.0050) < 0.0001
    # the thirteen 3x3 layers of VGG-16 at batch 256 (the 128-bit classifier adds the rest of the 5.13 T)
    vgg = [l for l in w["vgg16"]["layers"] if l[3] == 3]
    assert len(vgg) == 13 and abs(bench.bitops_per_image(vgg) * 256 / 1e12 - 5.13) < 0.01
    # every ResNet stage halves the map and doubles the channels; strided and shortcut layers come in pairs
    for name in ("resnet18", "resnet34"):
        strided = [l for l in w[name]["layers"] if l[4] == 2]
        assert len(strided) == 6 and {l[3] for l in strided} == {1, 3}
    # every workload names a metric, a batch and a description; the CPU sample batch is bounded
    for name, wl in w.items():
        assert wl["metric"] and wl["batch"] >= 1 and wl["text"]
        assert 1 <= bench._sample_batch(wl) <= wl["batch"] or wl["kind"] == "linear"
    assert bench._sample_batch(w["resnet18"]) == 4
