// Generic binary heap over a random-access container (pico-ps/common/Heap.h:14-89; unused by the rest
// of the reference, kept for API parity; the controller uses it to pick least-loaded nodes).
#pragma once
#include <functional>
#include <utility>
#include <vector>

namespace psb {

template <class T, class Less = std::less<T>>
class Heap {
public:
    explicit Heap(Less less = Less()) : less_(less) {}
    bool empty() const { return v_.empty(); }
    size_t size() const { return v_.size(); }
    const T& top() const { return v_.front(); }
    void push(T x) {
        v_.push_back(std::move(x));
        size_t i = v_.size() - 1;
        while (i > 0) {
            size_t p = (i - 1) / 2;
            if (!less_(v_[i], v_[p])) break;
            std::swap(v_[i], v_[p]);
            i = p;
        }
    }
    T pop() {
        T out = std::move(v_.front());
        v_.front() = std::move(v_.back());
        v_.pop_back();
        size_t i = 0, n = v_.size();
        for (;;) {
            size_t l = 2 * i + 1, r = l + 1, m = i;
            if (l < n && less_(v_[l], v_[m])) m = l;
            if (r < n && less_(v_[r], v_[m])) m = r;
            if (m == i) break;
            std::swap(v_[i], v_[m]);
            i = m;
        }
        return out;
    }

private:
    std::vector<T> v_;
    Less less_;
};

}  // namespace psb
