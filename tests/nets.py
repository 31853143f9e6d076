"""Small networks shared by the CPU and GPU tests (built with the same builders
as the benchmark configurations)."""
from nebula_b200.workloads import NetBuilder, alexnet, dbn, lstm2, resnet50, rnn2, vgg16


def toy_convnet(batch=3):
    """Every layer kind of the convolutional networks, odd extents, 3-channel input."""
    b = NetBuilder("toy", batch, 3, 19, 17, bias_init="bias_n01")
    b.conv(32, 3, 1, 1, "leaky", bn=True).maxpool(2, 2, 0).conv(48, 5, 2, 2, "relu").maxpool(3, 2)
    b.conv(64, 1, 1, 0, "linear", bn=True).conv(64, 3, 1, 1, "leaky", bn=True).conv(64, 1, 1, 0, "linear")
    b.shortcut(3, "leaky").avgpool(2, 2, 0)
    b.connected(40, "tanh").dropout().connected(24, "logistic", bn=True).connected(10, "linear").softmax()
    return b.build()


def tiny_vgg(batch=4):
    return vgg16(batch=batch, height=32, width=32, fc=128, classes=10, widths=(32, 32, 64, 64, 64))


def mid_vgg(batch=2):
    """Big enough (56x56, 64/128 channels) for the 3x3 halo kernel and its fused pooling."""
    return vgg16(batch=batch, height=56, width=56, fc=64, classes=10, widths=(64, 128, 64, 64, 64))


def tiny_resnet(batch=2):
    return resnet50(batch=batch, height=64, width=64, base=32, blocks=(2, 2, 2, 2), classes=10)


def tiny_lstm(batch=4, time_steps=6):
    return lstm2(batch=batch, time_steps=time_steps, input_size=64, hidden=32, classes=50)


def tiny_rnn(batch=4, time_steps=5):
    """Two [rnn] layers (tanh, then batch-normalised leaky) and a projection, wide enough for the tensor-core path."""
    b = NetBuilder("tiny_rnn", batch, input_size=64, time_steps=time_steps, bias_init="bias_n01")
    b.rnn(64, "tanh", bound=0.2).rnn(32, "leaky", bn=True, bound=0.2).connected(50, "linear", init="uniform", bound=0.2)
    return b.build("normal")


def tiny_lstm_act(batch=4, time_steps=5):
    """LSTM layers whose gate layers carry a non-linear section activation."""
    b = NetBuilder("tiny_lstm_act", batch, input_size=64, time_steps=time_steps, bias_init="bias_n01")
    b.lstm(32, act="tanh", bound=0.2).lstm(32, act="leaky", bn=True, bound=0.2)
    b.connected(50, "linear", init="uniform", bound=0.2)
    return b.build("normal")


def tiny_dbn(batch=6):
    return dbn(batch=batch, height=8, width=8, channels=3, hidden=(96, 64, 32), classes=10)


def small_alexnet(batch=2):
    return alexnet(batch=batch)


NETS = {"toy": toy_convnet, "tiny_vgg": tiny_vgg, "mid_vgg": mid_vgg, "tiny_resnet": tiny_resnet, "tiny_lstm": tiny_lstm,
        "tiny_rnn": tiny_rnn, "tiny_lstm_act": tiny_lstm_act, "tiny_dbn": tiny_dbn}
