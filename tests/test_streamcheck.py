"""The stream-order checker (a debug aid against cross-stream races on shared buffers), on symbolic streams."""
import pytest

from pippy_b200.utils.streamcheck import StreamOrderError, StreamTracker


def test_reduction_on_a_side_stream_must_be_waited_for():
    t = StreamTracker()
    t.write("grad", "compute")                 # backward produced the gradients
    t.ordered("compute", "side")               # side stream waits for an event recorded on compute
    t.write("grad", "side")                    # the all-reduce rewrites them there
    with pytest.raises(StreamOrderError, match="without waiting for its writer"):
        t.read("grad", "compute")              # scaling / optimizer before finish(): the race this tool is for
    t.ordered("side", "compute")               # finish(): compute waits for the reduction's event
    t.read("grad", "compute")
    t.write("grad", "compute")


def test_side_stream_launch_without_waiting_for_the_producer():
    t = StreamTracker()
    t.write("grad", "compute")
    with pytest.raises(StreamOrderError, match="previous writer"):
        t.write("grad", "side")


def test_overwrite_while_another_stream_may_still_read():
    t = StreamTracker()
    t.write("act", "compute")
    t.ordered("compute", "send")
    t.read("act", "send")                      # a send reads the activation on the communicator's stream
    with pytest.raises(StreamOrderError, match="may still read"):
        t.write("act", "compute")              # the buffer is reused before the send was waited for
    t.ordered("send", "compute")
    t.write("act", "compute")


def test_ordering_is_transitive_and_only_covers_earlier_work():
    t = StreamTracker()
    t.write("x", "a")
    t.ordered("a", "b")
    t.ordered("b", "c")                        # c is after b, which was after a's write
    t.read("x", "c")
    t2 = StreamTracker()
    t2.write("x", "a")
    t2.ordered("a", "b")
    t2.ordered("b", "a")
    t2.write("x", "a")                         # b was ordered after a's FIRST write only
    with pytest.raises(StreamOrderError):
        t2.read("x", "b")
