// Hook for reductions that can fold four packed 1-byte elements at once: the kernels of
// reduce.cuh test word_accum<R, T>::ok and, when set, call word_accum<R, T>::apply(r, acc, word);
// the specialisations sit beside the reductions in ops_reduce.cuh.
#pragma once
namespace sd {
template <class R, class T> struct word_accum { static constexpr bool ok = false; };
}
