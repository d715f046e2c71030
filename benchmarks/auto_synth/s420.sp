* s420 (s420: 16-bit fractional multiplier control): 240 gates, 1824 transistors
VDD vdd 0 DC 1.8
VIN0 ni0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 ni1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 ni2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 ni3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 ni4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 ni5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 ni6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 ni7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 nq0 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 nq1 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 nq2 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 nq3 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nq4 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nq5 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nq6 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nq7 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nq8 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nq9 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nq10 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nq11 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nq12 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nq13 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nq14 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nq15 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
CT1 t1 0 0.1f
CT2 t2 0 0.1f
CT3 t3 0 0.1f
M1 t1 nq0 vdd vdd pch w=2u l=180n
M2 t1 ni0 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M3 t1 nq0 t4 0 nch w=1u l=180n
M4 t4 ni0 0 0 nch w=1u l=180n
M5 t2 nq0 vdd vdd pch w=2u l=180n
M6 t2 t1 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M7 t2 nq0 t5 0 nch w=1u l=180n
M8 t5 t1 0 0 nch w=1u l=180n
M9 t3 ni0 vdd vdd pch w=2u l=180n
M10 t3 t1 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M11 t3 ni0 t6 0 nch w=1u l=180n
M12 t6 t1 0 0 nch w=1u l=180n
M13 nw1 t2 vdd vdd pch w=2u l=180n
M14 nw1 t3 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M15 nw1 t2 t7 0 nch w=1u l=180n
M16 t7 t3 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
CT8 t8 0 0.1f
M17 t8 ni0 vdd vdd pch w=2u l=180n
M18 t8 nq0 vdd vdd pch w=2u l=180n
CT9 t9 0 0.1f
M19 t8 ni0 t9 0 nch w=1u l=180n
M20 t9 nq0 0 0 nch w=1u l=180n
M21 nw2 t8 vdd vdd pch w=2u l=180n
M22 nw2 t8 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
CT10 t10 0 0.1f
CT11 t11 0 0.1f
CT12 t12 0 0.1f
M23 t10 nq1 vdd vdd pch w=2u l=180n
M24 t10 nw2 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M25 t10 nq1 t13 0 nch w=1u l=180n
M26 t13 nw2 0 0 nch w=1u l=180n
M27 t11 nq1 vdd vdd pch w=2u l=180n
M28 t11 t10 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M29 t11 nq1 t14 0 nch w=1u l=180n
M30 t14 t10 0 0 nch w=1u l=180n
M31 t12 nw2 vdd vdd pch w=2u l=180n
M32 t12 t10 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M33 t12 nw2 t15 0 nch w=1u l=180n
M34 t15 t10 0 0 nch w=1u l=180n
M35 nw3 t11 vdd vdd pch w=2u l=180n
M36 nw3 t12 vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M37 nw3 t11 t16 0 nch w=1u l=180n
M38 t16 t12 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
CT17 t17 0 0.1f
M39 t17 nw2 vdd vdd pch w=2u l=180n
M40 t17 nq1 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M41 t17 nw2 t18 0 nch w=1u l=180n
M42 t18 nq1 0 0 nch w=1u l=180n
M43 nw4 t17 vdd vdd pch w=2u l=180n
M44 nw4 t17 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
CT19 t19 0 0.1f
CT20 t20 0 0.1f
CT21 t21 0 0.1f
M45 t19 nq2 vdd vdd pch w=2u l=180n
M46 t19 nw4 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M47 t19 nq2 t22 0 nch w=1u l=180n
M48 t22 nw4 0 0 nch w=1u l=180n
M49 t20 nq2 vdd vdd pch w=2u l=180n
M50 t20 t19 vdd vdd pch w=2u l=180n
CT23 t23 0 0.1f
M51 t20 nq2 t23 0 nch w=1u l=180n
M52 t23 t19 0 0 nch w=1u l=180n
M53 t21 nw4 vdd vdd pch w=2u l=180n
M54 t21 t19 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M55 t21 nw4 t24 0 nch w=1u l=180n
M56 t24 t19 0 0 nch w=1u l=180n
M57 nw5 t20 vdd vdd pch w=2u l=180n
M58 nw5 t21 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M59 nw5 t20 t25 0 nch w=1u l=180n
M60 t25 t21 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
CT26 t26 0 0.1f
M61 t26 nw4 vdd vdd pch w=2u l=180n
M62 t26 nq2 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M63 t26 nw4 t27 0 nch w=1u l=180n
M64 t27 nq2 0 0 nch w=1u l=180n
M65 nw6 t26 vdd vdd pch w=2u l=180n
M66 nw6 t26 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
CT28 t28 0 0.1f
CT29 t29 0 0.1f
CT30 t30 0 0.1f
M67 t28 nq3 vdd vdd pch w=2u l=180n
M68 t28 nw6 vdd vdd pch w=2u l=180n
CT31 t31 0 0.1f
M69 t28 nq3 t31 0 nch w=1u l=180n
M70 t31 nw6 0 0 nch w=1u l=180n
M71 t29 nq3 vdd vdd pch w=2u l=180n
M72 t29 t28 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M73 t29 nq3 t32 0 nch w=1u l=180n
M74 t32 t28 0 0 nch w=1u l=180n
M75 t30 nw6 vdd vdd pch w=2u l=180n
M76 t30 t28 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M77 t30 nw6 t33 0 nch w=1u l=180n
M78 t33 t28 0 0 nch w=1u l=180n
M79 nw7 t29 vdd vdd pch w=2u l=180n
M80 nw7 t30 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M81 nw7 t29 t34 0 nch w=1u l=180n
M82 t34 t30 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
CT35 t35 0 0.1f
M83 t35 nw6 vdd vdd pch w=2u l=180n
M84 t35 nq3 vdd vdd pch w=2u l=180n
CT36 t36 0 0.1f
M85 t35 nw6 t36 0 nch w=1u l=180n
M86 t36 nq3 0 0 nch w=1u l=180n
M87 nw8 t35 vdd vdd pch w=2u l=180n
M88 nw8 t35 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
CT37 t37 0 0.1f
CT38 t38 0 0.1f
CT39 t39 0 0.1f
M89 t37 nq4 vdd vdd pch w=2u l=180n
M90 t37 nw8 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M91 t37 nq4 t40 0 nch w=1u l=180n
M92 t40 nw8 0 0 nch w=1u l=180n
M93 t38 nq4 vdd vdd pch w=2u l=180n
M94 t38 t37 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M95 t38 nq4 t41 0 nch w=1u l=180n
M96 t41 t37 0 0 nch w=1u l=180n
M97 t39 nw8 vdd vdd pch w=2u l=180n
M98 t39 t37 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M99 t39 nw8 t42 0 nch w=1u l=180n
M100 t42 t37 0 0 nch w=1u l=180n
M101 nw9 t38 vdd vdd pch w=2u l=180n
M102 nw9 t39 vdd vdd pch w=2u l=180n
CT43 t43 0 0.1f
M103 nw9 t38 t43 0 nch w=1u l=180n
M104 t43 t39 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
CT44 t44 0 0.1f
M105 t44 nw8 vdd vdd pch w=2u l=180n
M106 t44 nq4 vdd vdd pch w=2u l=180n
CT45 t45 0 0.1f
M107 t44 nw8 t45 0 nch w=1u l=180n
M108 t45 nq4 0 0 nch w=1u l=180n
M109 nw10 t44 vdd vdd pch w=2u l=180n
M110 nw10 t44 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
CT46 t46 0 0.1f
CT47 t47 0 0.1f
CT48 t48 0 0.1f
M111 t46 nq5 vdd vdd pch w=2u l=180n
M112 t46 nw10 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M113 t46 nq5 t49 0 nch w=1u l=180n
M114 t49 nw10 0 0 nch w=1u l=180n
M115 t47 nq5 vdd vdd pch w=2u l=180n
M116 t47 t46 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M117 t47 nq5 t50 0 nch w=1u l=180n
M118 t50 t46 0 0 nch w=1u l=180n
M119 t48 nw10 vdd vdd pch w=2u l=180n
M120 t48 t46 vdd vdd pch w=2u l=180n
CT51 t51 0 0.1f
M121 t48 nw10 t51 0 nch w=1u l=180n
M122 t51 t46 0 0 nch w=1u l=180n
M123 nw11 t47 vdd vdd pch w=2u l=180n
M124 nw11 t48 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M125 nw11 t47 t52 0 nch w=1u l=180n
M126 t52 t48 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
CT53 t53 0 0.1f
M127 t53 nw10 vdd vdd pch w=2u l=180n
M128 t53 nq5 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M129 t53 nw10 t54 0 nch w=1u l=180n
M130 t54 nq5 0 0 nch w=1u l=180n
M131 nw12 t53 vdd vdd pch w=2u l=180n
M132 nw12 t53 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
CT55 t55 0 0.1f
CT56 t56 0 0.1f
CT57 t57 0 0.1f
M133 t55 nq6 vdd vdd pch w=2u l=180n
M134 t55 nw12 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M135 t55 nq6 t58 0 nch w=1u l=180n
M136 t58 nw12 0 0 nch w=1u l=180n
M137 t56 nq6 vdd vdd pch w=2u l=180n
M138 t56 t55 vdd vdd pch w=2u l=180n
CT59 t59 0 0.1f
M139 t56 nq6 t59 0 nch w=1u l=180n
M140 t59 t55 0 0 nch w=1u l=180n
M141 t57 nw12 vdd vdd pch w=2u l=180n
M142 t57 t55 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M143 t57 nw12 t60 0 nch w=1u l=180n
M144 t60 t55 0 0 nch w=1u l=180n
M145 nw13 t56 vdd vdd pch w=2u l=180n
M146 nw13 t57 vdd vdd pch w=2u l=180n
CT61 t61 0 0.1f
M147 nw13 t56 t61 0 nch w=1u l=180n
M148 t61 t57 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
CT62 t62 0 0.1f
M149 t62 nw12 vdd vdd pch w=2u l=180n
M150 t62 nq6 vdd vdd pch w=2u l=180n
CT63 t63 0 0.1f
M151 t62 nw12 t63 0 nch w=1u l=180n
M152 t63 nq6 0 0 nch w=1u l=180n
M153 nw14 t62 vdd vdd pch w=2u l=180n
M154 nw14 t62 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
CT64 t64 0 0.1f
CT65 t65 0 0.1f
CT66 t66 0 0.1f
M155 t64 nq7 vdd vdd pch w=2u l=180n
M156 t64 nw14 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M157 t64 nq7 t67 0 nch w=1u l=180n
M158 t67 nw14 0 0 nch w=1u l=180n
M159 t65 nq7 vdd vdd pch w=2u l=180n
M160 t65 t64 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M161 t65 nq7 t68 0 nch w=1u l=180n
M162 t68 t64 0 0 nch w=1u l=180n
M163 t66 nw14 vdd vdd pch w=2u l=180n
M164 t66 t64 vdd vdd pch w=2u l=180n
CT69 t69 0 0.1f
M165 t66 nw14 t69 0 nch w=1u l=180n
M166 t69 t64 0 0 nch w=1u l=180n
M167 nw15 t65 vdd vdd pch w=2u l=180n
M168 nw15 t66 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M169 nw15 t65 t70 0 nch w=1u l=180n
M170 t70 t66 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
CT71 t71 0 0.1f
M171 t71 nw14 vdd vdd pch w=2u l=180n
M172 t71 nq7 vdd vdd pch w=2u l=180n
CT72 t72 0 0.1f
M173 t71 nw14 t72 0 nch w=1u l=180n
M174 t72 nq7 0 0 nch w=1u l=180n
M175 nw16 t71 vdd vdd pch w=2u l=180n
M176 nw16 t71 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
CT73 t73 0 0.1f
CT74 t74 0 0.1f
CT75 t75 0 0.1f
M177 t73 nq8 vdd vdd pch w=2u l=180n
M178 t73 nw16 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M179 t73 nq8 t76 0 nch w=1u l=180n
M180 t76 nw16 0 0 nch w=1u l=180n
M181 t74 nq8 vdd vdd pch w=2u l=180n
M182 t74 t73 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M183 t74 nq8 t77 0 nch w=1u l=180n
M184 t77 t73 0 0 nch w=1u l=180n
M185 t75 nw16 vdd vdd pch w=2u l=180n
M186 t75 t73 vdd vdd pch w=2u l=180n
CT78 t78 0 0.1f
M187 t75 nw16 t78 0 nch w=1u l=180n
M188 t78 t73 0 0 nch w=1u l=180n
M189 nw17 t74 vdd vdd pch w=2u l=180n
M190 nw17 t75 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M191 nw17 t74 t79 0 nch w=1u l=180n
M192 t79 t75 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
CT80 t80 0 0.1f
M193 t80 nw16 vdd vdd pch w=2u l=180n
M194 t80 nq8 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M195 t80 nw16 t81 0 nch w=1u l=180n
M196 t81 nq8 0 0 nch w=1u l=180n
M197 nw18 t80 vdd vdd pch w=2u l=180n
M198 nw18 t80 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
CT82 t82 0 0.1f
CT83 t83 0 0.1f
CT84 t84 0 0.1f
M199 t82 nq9 vdd vdd pch w=2u l=180n
M200 t82 nw18 vdd vdd pch w=2u l=180n
CT85 t85 0 0.1f
M201 t82 nq9 t85 0 nch w=1u l=180n
M202 t85 nw18 0 0 nch w=1u l=180n
M203 t83 nq9 vdd vdd pch w=2u l=180n
M204 t83 t82 vdd vdd pch w=2u l=180n
CT86 t86 0 0.1f
M205 t83 nq9 t86 0 nch w=1u l=180n
M206 t86 t82 0 0 nch w=1u l=180n
M207 t84 nw18 vdd vdd pch w=2u l=180n
M208 t84 t82 vdd vdd pch w=2u l=180n
CT87 t87 0 0.1f
M209 t84 nw18 t87 0 nch w=1u l=180n
M210 t87 t82 0 0 nch w=1u l=180n
M211 nw19 t83 vdd vdd pch w=2u l=180n
M212 nw19 t84 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M213 nw19 t83 t88 0 nch w=1u l=180n
M214 t88 t84 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
CT89 t89 0 0.1f
M215 t89 nw18 vdd vdd pch w=2u l=180n
M216 t89 nq9 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M217 t89 nw18 t90 0 nch w=1u l=180n
M218 t90 nq9 0 0 nch w=1u l=180n
M219 nw20 t89 vdd vdd pch w=2u l=180n
M220 nw20 t89 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
CT91 t91 0 0.1f
CT92 t92 0 0.1f
CT93 t93 0 0.1f
M221 t91 nq10 vdd vdd pch w=2u l=180n
M222 t91 nw20 vdd vdd pch w=2u l=180n
CT94 t94 0 0.1f
M223 t91 nq10 t94 0 nch w=1u l=180n
M224 t94 nw20 0 0 nch w=1u l=180n
M225 t92 nq10 vdd vdd pch w=2u l=180n
M226 t92 t91 vdd vdd pch w=2u l=180n
CT95 t95 0 0.1f
M227 t92 nq10 t95 0 nch w=1u l=180n
M228 t95 t91 0 0 nch w=1u l=180n
M229 t93 nw20 vdd vdd pch w=2u l=180n
M230 t93 t91 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M231 t93 nw20 t96 0 nch w=1u l=180n
M232 t96 t91 0 0 nch w=1u l=180n
M233 nw21 t92 vdd vdd pch w=2u l=180n
M234 nw21 t93 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M235 nw21 t92 t97 0 nch w=1u l=180n
M236 t97 t93 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
CT98 t98 0 0.1f
M237 t98 nw20 vdd vdd pch w=2u l=180n
M238 t98 nq10 vdd vdd pch w=2u l=180n
CT99 t99 0 0.1f
M239 t98 nw20 t99 0 nch w=1u l=180n
M240 t99 nq10 0 0 nch w=1u l=180n
M241 nw22 t98 vdd vdd pch w=2u l=180n
M242 nw22 t98 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
CT100 t100 0 0.1f
CT101 t101 0 0.1f
CT102 t102 0 0.1f
M243 t100 nq11 vdd vdd pch w=2u l=180n
M244 t100 nw22 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M245 t100 nq11 t103 0 nch w=1u l=180n
M246 t103 nw22 0 0 nch w=1u l=180n
M247 t101 nq11 vdd vdd pch w=2u l=180n
M248 t101 t100 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M249 t101 nq11 t104 0 nch w=1u l=180n
M250 t104 t100 0 0 nch w=1u l=180n
M251 t102 nw22 vdd vdd pch w=2u l=180n
M252 t102 t100 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M253 t102 nw22 t105 0 nch w=1u l=180n
M254 t105 t100 0 0 nch w=1u l=180n
M255 nw23 t101 vdd vdd pch w=2u l=180n
M256 nw23 t102 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M257 nw23 t101 t106 0 nch w=1u l=180n
M258 t106 t102 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
CT107 t107 0 0.1f
M259 t107 nw22 vdd vdd pch w=2u l=180n
M260 t107 nq11 vdd vdd pch w=2u l=180n
CT108 t108 0 0.1f
M261 t107 nw22 t108 0 nch w=1u l=180n
M262 t108 nq11 0 0 nch w=1u l=180n
M263 nw24 t107 vdd vdd pch w=2u l=180n
M264 nw24 t107 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
CT109 t109 0 0.1f
CT110 t110 0 0.1f
CT111 t111 0 0.1f
M265 t109 nq12 vdd vdd pch w=2u l=180n
M266 t109 nw24 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M267 t109 nq12 t112 0 nch w=1u l=180n
M268 t112 nw24 0 0 nch w=1u l=180n
M269 t110 nq12 vdd vdd pch w=2u l=180n
M270 t110 t109 vdd vdd pch w=2u l=180n
CT113 t113 0 0.1f
M271 t110 nq12 t113 0 nch w=1u l=180n
M272 t113 t109 0 0 nch w=1u l=180n
M273 t111 nw24 vdd vdd pch w=2u l=180n
M274 t111 t109 vdd vdd pch w=2u l=180n
CT114 t114 0 0.1f
M275 t111 nw24 t114 0 nch w=1u l=180n
M276 t114 t109 0 0 nch w=1u l=180n
M277 nw25 t110 vdd vdd pch w=2u l=180n
M278 nw25 t111 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M279 nw25 t110 t115 0 nch w=1u l=180n
M280 t115 t111 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
CT116 t116 0 0.1f
M281 t116 nw24 vdd vdd pch w=2u l=180n
M282 t116 nq12 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M283 t116 nw24 t117 0 nch w=1u l=180n
M284 t117 nq12 0 0 nch w=1u l=180n
M285 nw26 t116 vdd vdd pch w=2u l=180n
M286 nw26 t116 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
CT118 t118 0 0.1f
CT119 t119 0 0.1f
CT120 t120 0 0.1f
M287 t118 nq13 vdd vdd pch w=2u l=180n
M288 t118 nw26 vdd vdd pch w=2u l=180n
CT121 t121 0 0.1f
M289 t118 nq13 t121 0 nch w=1u l=180n
M290 t121 nw26 0 0 nch w=1u l=180n
M291 t119 nq13 vdd vdd pch w=2u l=180n
M292 t119 t118 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M293 t119 nq13 t122 0 nch w=1u l=180n
M294 t122 t118 0 0 nch w=1u l=180n
M295 t120 nw26 vdd vdd pch w=2u l=180n
M296 t120 t118 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M297 t120 nw26 t123 0 nch w=1u l=180n
M298 t123 t118 0 0 nch w=1u l=180n
M299 nw27 t119 vdd vdd pch w=2u l=180n
M300 nw27 t120 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M301 nw27 t119 t124 0 nch w=1u l=180n
M302 t124 t120 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
CT125 t125 0 0.1f
M303 t125 nw26 vdd vdd pch w=2u l=180n
M304 t125 nq13 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M305 t125 nw26 t126 0 nch w=1u l=180n
M306 t126 nq13 0 0 nch w=1u l=180n
M307 nw28 t125 vdd vdd pch w=2u l=180n
M308 nw28 t125 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
CT127 t127 0 0.1f
CT128 t128 0 0.1f
CT129 t129 0 0.1f
M309 t127 nq14 vdd vdd pch w=2u l=180n
M310 t127 nw28 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M311 t127 nq14 t130 0 nch w=1u l=180n
M312 t130 nw28 0 0 nch w=1u l=180n
M313 t128 nq14 vdd vdd pch w=2u l=180n
M314 t128 t127 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M315 t128 nq14 t131 0 nch w=1u l=180n
M316 t131 t127 0 0 nch w=1u l=180n
M317 t129 nw28 vdd vdd pch w=2u l=180n
M318 t129 t127 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M319 t129 nw28 t132 0 nch w=1u l=180n
M320 t132 t127 0 0 nch w=1u l=180n
M321 nw29 t128 vdd vdd pch w=2u l=180n
M322 nw29 t129 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M323 nw29 t128 t133 0 nch w=1u l=180n
M324 t133 t129 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
CT134 t134 0 0.1f
M325 t134 nw28 vdd vdd pch w=2u l=180n
M326 t134 nq14 vdd vdd pch w=2u l=180n
CT135 t135 0 0.1f
M327 t134 nw28 t135 0 nch w=1u l=180n
M328 t135 nq14 0 0 nch w=1u l=180n
M329 nw30 t134 vdd vdd pch w=2u l=180n
M330 nw30 t134 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
CT136 t136 0 0.1f
CT137 t137 0 0.1f
CT138 t138 0 0.1f
M331 t136 nq15 vdd vdd pch w=2u l=180n
M332 t136 nw30 vdd vdd pch w=2u l=180n
CT139 t139 0 0.1f
M333 t136 nq15 t139 0 nch w=1u l=180n
M334 t139 nw30 0 0 nch w=1u l=180n
M335 t137 nq15 vdd vdd pch w=2u l=180n
M336 t137 t136 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M337 t137 nq15 t140 0 nch w=1u l=180n
M338 t140 t136 0 0 nch w=1u l=180n
M339 t138 nw30 vdd vdd pch w=2u l=180n
M340 t138 t136 vdd vdd pch w=2u l=180n
CT141 t141 0 0.1f
M341 t138 nw30 t141 0 nch w=1u l=180n
M342 t141 t136 0 0 nch w=1u l=180n
M343 nw31 t137 vdd vdd pch w=2u l=180n
M344 nw31 t138 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M345 nw31 t137 t142 0 nch w=1u l=180n
M346 t142 t138 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
CT143 t143 0 0.1f
M347 t143 nw30 vdd vdd pch w=2u l=180n
M348 t143 nq15 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M349 t143 nw30 t144 0 nch w=1u l=180n
M350 t144 nq15 0 0 nch w=1u l=180n
M351 nw32 t143 vdd vdd pch w=2u l=180n
M352 nw32 t143 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
M353 nw33 nq1 vdd vdd pch w=2u l=180n
M354 nw33 nq3 vdd vdd pch w=2u l=180n
CT145 t145 0 0.1f
M355 nw33 nq1 t145 0 nch w=1u l=180n
M356 t145 nq3 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
M357 nw34 nq8 0 0 nch w=1u l=180n
M358 nw34 nq14 0 0 nch w=1u l=180n
CT146 t146 0 0.1f
M359 t146 nq8 vdd vdd pch w=2u l=180n
M360 nw34 nq14 t146 vdd pch w=2u l=180n
Cnw34 nw34 0 2f
CT147 t147 0 0.1f
M361 t147 nq15 vdd vdd pch w=2u l=180n
M362 t147 nw34 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M363 t147 nq15 t148 0 nch w=1u l=180n
M364 t148 nw34 0 0 nch w=1u l=180n
M365 nw35 t147 vdd vdd pch w=2u l=180n
M366 nw35 t147 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
CT149 t149 0 0.1f
M367 t149 ni6 0 0 nch w=1u l=180n
M368 t149 nq9 0 0 nch w=1u l=180n
CT150 t150 0 0.1f
M369 t150 ni6 vdd vdd pch w=2u l=180n
M370 t149 nq9 t150 vdd pch w=2u l=180n
M371 nw36 t149 vdd vdd pch w=2u l=180n
M372 nw36 t149 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
CT151 t151 0 0.1f
CT152 t152 0 0.1f
CT153 t153 0 0.1f
M373 t151 nq1 vdd vdd pch w=2u l=180n
M374 t151 ni3 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M375 t151 nq1 t154 0 nch w=1u l=180n
M376 t154 ni3 0 0 nch w=1u l=180n
M377 t152 nq1 vdd vdd pch w=2u l=180n
M378 t152 t151 vdd vdd pch w=2u l=180n
CT155 t155 0 0.1f
M379 t152 nq1 t155 0 nch w=1u l=180n
M380 t155 t151 0 0 nch w=1u l=180n
M381 t153 ni3 vdd vdd pch w=2u l=180n
M382 t153 t151 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M383 t153 ni3 t156 0 nch w=1u l=180n
M384 t156 t151 0 0 nch w=1u l=180n
M385 nw37 t152 vdd vdd pch w=2u l=180n
M386 nw37 t153 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M387 nw37 t152 t157 0 nch w=1u l=180n
M388 t157 t153 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
M389 nw38 nq7 vdd vdd pch w=2u l=180n
M390 nw38 nq0 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M391 nw38 nq7 t158 0 nch w=1u l=180n
M392 t158 nq0 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
M393 nw39 nq13 0 0 nch w=1u l=180n
M394 nw39 nq9 0 0 nch w=1u l=180n
CT159 t159 0 0.1f
M395 t159 nq13 vdd vdd pch w=2u l=180n
M396 nw39 nq9 t159 vdd pch w=2u l=180n
Cnw39 nw39 0 2f
CT160 t160 0 0.1f
M397 t160 ni3 vdd vdd pch w=2u l=180n
M398 t160 ni2 vdd vdd pch w=2u l=180n
CT161 t161 0 0.1f
M399 t160 ni3 t161 0 nch w=1u l=180n
M400 t161 ni2 0 0 nch w=1u l=180n
M401 nw40 t160 vdd vdd pch w=2u l=180n
M402 nw40 t160 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
CT162 t162 0 0.1f
M403 t162 nw34 0 0 nch w=1u l=180n
M404 t162 nw36 0 0 nch w=1u l=180n
CT163 t163 0 0.1f
M405 t163 nw34 vdd vdd pch w=2u l=180n
M406 t162 nw36 t163 vdd pch w=2u l=180n
M407 nw41 t162 vdd vdd pch w=2u l=180n
M408 nw41 t162 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
CT164 t164 0 0.1f
CT165 t165 0 0.1f
CT166 t166 0 0.1f
M409 t164 nw40 vdd vdd pch w=2u l=180n
M410 t164 nq3 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M411 t164 nw40 t167 0 nch w=1u l=180n
M412 t167 nq3 0 0 nch w=1u l=180n
M413 t165 nw40 vdd vdd pch w=2u l=180n
M414 t165 t164 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M415 t165 nw40 t168 0 nch w=1u l=180n
M416 t168 t164 0 0 nch w=1u l=180n
M417 t166 nq3 vdd vdd pch w=2u l=180n
M418 t166 t164 vdd vdd pch w=2u l=180n
CT169 t169 0 0.1f
M419 t166 nq3 t169 0 nch w=1u l=180n
M420 t169 t164 0 0 nch w=1u l=180n
M421 nw42 t165 vdd vdd pch w=2u l=180n
M422 nw42 t166 vdd vdd pch w=2u l=180n
CT170 t170 0 0.1f
M423 nw42 t165 t170 0 nch w=1u l=180n
M424 t170 t166 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
M425 nw43 nq3 vdd vdd pch w=2u l=180n
M426 nw43 nq11 vdd vdd pch w=2u l=180n
CT171 t171 0 0.1f
M427 nw43 nq3 t171 0 nch w=1u l=180n
M428 t171 nq11 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
M429 nw44 nq8 0 0 nch w=1u l=180n
M430 nw44 ni3 0 0 nch w=1u l=180n
CT172 t172 0 0.1f
M431 t172 nq8 vdd vdd pch w=2u l=180n
M432 nw44 ni3 t172 vdd pch w=2u l=180n
Cnw44 nw44 0 2f
CT173 t173 0 0.1f
M433 t173 nq13 vdd vdd pch w=2u l=180n
M434 t173 nw36 vdd vdd pch w=2u l=180n
CT174 t174 0 0.1f
M435 t173 nq13 t174 0 nch w=1u l=180n
M436 t174 nw36 0 0 nch w=1u l=180n
M437 nw45 t173 vdd vdd pch w=2u l=180n
M438 nw45 t173 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
CT175 t175 0 0.1f
M439 t175 ni2 0 0 nch w=1u l=180n
M440 t175 nw44 0 0 nch w=1u l=180n
CT176 t176 0 0.1f
M441 t176 ni2 vdd vdd pch w=2u l=180n
M442 t175 nw44 t176 vdd pch w=2u l=180n
M443 nw46 t175 vdd vdd pch w=2u l=180n
M444 nw46 t175 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
CT177 t177 0 0.1f
CT178 t178 0 0.1f
CT179 t179 0 0.1f
M445 t177 ni7 vdd vdd pch w=2u l=180n
M446 t177 nq5 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M447 t177 ni7 t180 0 nch w=1u l=180n
M448 t180 nq5 0 0 nch w=1u l=180n
M449 t178 ni7 vdd vdd pch w=2u l=180n
M450 t178 t177 vdd vdd pch w=2u l=180n
CT181 t181 0 0.1f
M451 t178 ni7 t181 0 nch w=1u l=180n
M452 t181 t177 0 0 nch w=1u l=180n
M453 t179 nq5 vdd vdd pch w=2u l=180n
M454 t179 t177 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M455 t179 nq5 t182 0 nch w=1u l=180n
M456 t182 t177 0 0 nch w=1u l=180n
M457 nw47 t178 vdd vdd pch w=2u l=180n
M458 nw47 t179 vdd vdd pch w=2u l=180n
CT183 t183 0 0.1f
M459 nw47 t178 t183 0 nch w=1u l=180n
M460 t183 t179 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
M461 nw48 nw37 vdd vdd pch w=2u l=180n
M462 nw48 nq12 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M463 nw48 nw37 t184 0 nch w=1u l=180n
M464 t184 nq12 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
M465 nw49 nw42 0 0 nch w=1u l=180n
M466 nw49 ni3 0 0 nch w=1u l=180n
CT185 t185 0 0.1f
M467 t185 nw42 vdd vdd pch w=2u l=180n
M468 nw49 ni3 t185 vdd pch w=2u l=180n
Cnw49 nw49 0 2f
CT186 t186 0 0.1f
M469 t186 nw47 vdd vdd pch w=2u l=180n
M470 t186 nw35 vdd vdd pch w=2u l=180n
CT187 t187 0 0.1f
M471 t186 nw47 t187 0 nch w=1u l=180n
M472 t187 nw35 0 0 nch w=1u l=180n
M473 nw50 t186 vdd vdd pch w=2u l=180n
M474 nw50 t186 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
CT188 t188 0 0.1f
M475 t188 nq1 0 0 nch w=1u l=180n
M476 t188 nw42 0 0 nch w=1u l=180n
CT189 t189 0 0.1f
M477 t189 nq1 vdd vdd pch w=2u l=180n
M478 t188 nw42 t189 vdd pch w=2u l=180n
M479 nw51 t188 vdd vdd pch w=2u l=180n
M480 nw51 t188 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
CT190 t190 0 0.1f
CT191 t191 0 0.1f
CT192 t192 0 0.1f
M481 t190 nq5 vdd vdd pch w=2u l=180n
M482 t190 nw49 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M483 t190 nq5 t193 0 nch w=1u l=180n
M484 t193 nw49 0 0 nch w=1u l=180n
M485 t191 nq5 vdd vdd pch w=2u l=180n
M486 t191 t190 vdd vdd pch w=2u l=180n
CT194 t194 0 0.1f
M487 t191 nq5 t194 0 nch w=1u l=180n
M488 t194 t190 0 0 nch w=1u l=180n
M489 t192 nw49 vdd vdd pch w=2u l=180n
M490 t192 t190 vdd vdd pch w=2u l=180n
CT195 t195 0 0.1f
M491 t192 nw49 t195 0 nch w=1u l=180n
M492 t195 t190 0 0 nch w=1u l=180n
M493 nw52 t191 vdd vdd pch w=2u l=180n
M494 nw52 t192 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M495 nw52 t191 t196 0 nch w=1u l=180n
M496 t196 t192 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M497 nw53 nq9 vdd vdd pch w=2u l=180n
M498 nw53 nq3 vdd vdd pch w=2u l=180n
CT197 t197 0 0.1f
M499 nw53 nq9 t197 0 nch w=1u l=180n
M500 t197 nq3 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
M501 nw54 nq13 0 0 nch w=1u l=180n
M502 nw54 nq9 0 0 nch w=1u l=180n
CT198 t198 0 0.1f
M503 t198 nq13 vdd vdd pch w=2u l=180n
M504 nw54 nq9 t198 vdd pch w=2u l=180n
Cnw54 nw54 0 2f
CT199 t199 0 0.1f
M505 t199 ni1 vdd vdd pch w=2u l=180n
M506 t199 nq15 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M507 t199 ni1 t200 0 nch w=1u l=180n
M508 t200 nq15 0 0 nch w=1u l=180n
M509 nw55 t199 vdd vdd pch w=2u l=180n
M510 nw55 t199 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
CT201 t201 0 0.1f
M511 t201 ni5 0 0 nch w=1u l=180n
M512 t201 ni6 0 0 nch w=1u l=180n
CT202 t202 0 0.1f
M513 t202 ni5 vdd vdd pch w=2u l=180n
M514 t201 ni6 t202 vdd pch w=2u l=180n
M515 nw56 t201 vdd vdd pch w=2u l=180n
M516 nw56 t201 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
CT203 t203 0 0.1f
CT204 t204 0 0.1f
CT205 t205 0 0.1f
M517 t203 nw34 vdd vdd pch w=2u l=180n
M518 t203 nw36 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M519 t203 nw34 t206 0 nch w=1u l=180n
M520 t206 nw36 0 0 nch w=1u l=180n
M521 t204 nw34 vdd vdd pch w=2u l=180n
M522 t204 t203 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M523 t204 nw34 t207 0 nch w=1u l=180n
M524 t207 t203 0 0 nch w=1u l=180n
M525 t205 nw36 vdd vdd pch w=2u l=180n
M526 t205 t203 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M527 t205 nw36 t208 0 nch w=1u l=180n
M528 t208 t203 0 0 nch w=1u l=180n
M529 nw57 t204 vdd vdd pch w=2u l=180n
M530 nw57 t205 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M531 nw57 t204 t209 0 nch w=1u l=180n
M532 t209 t205 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
M533 nw58 nw38 vdd vdd pch w=2u l=180n
M534 nw58 nw42 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M535 nw58 nw38 t210 0 nch w=1u l=180n
M536 t210 nw42 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
M537 nw59 nw42 0 0 nch w=1u l=180n
M538 nw59 nw48 0 0 nch w=1u l=180n
CT211 t211 0 0.1f
M539 t211 nw42 vdd vdd pch w=2u l=180n
M540 nw59 nw48 t211 vdd pch w=2u l=180n
Cnw59 nw59 0 2f
CT212 t212 0 0.1f
M541 t212 nw46 vdd vdd pch w=2u l=180n
M542 t212 nw54 vdd vdd pch w=2u l=180n
CT213 t213 0 0.1f
M543 t212 nw46 t213 0 nch w=1u l=180n
M544 t213 nw54 0 0 nch w=1u l=180n
M545 nw60 t212 vdd vdd pch w=2u l=180n
M546 nw60 t212 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
CT214 t214 0 0.1f
M547 t214 nw50 0 0 nch w=1u l=180n
M548 t214 nw60 0 0 nch w=1u l=180n
CT215 t215 0 0.1f
M549 t215 nw50 vdd vdd pch w=2u l=180n
M550 t214 nw60 t215 vdd pch w=2u l=180n
M551 nw61 t214 vdd vdd pch w=2u l=180n
M552 nw61 t214 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
CT216 t216 0 0.1f
CT217 t217 0 0.1f
CT218 t218 0 0.1f
M553 t216 nw54 vdd vdd pch w=2u l=180n
M554 t216 nq4 vdd vdd pch w=2u l=180n
CT219 t219 0 0.1f
M555 t216 nw54 t219 0 nch w=1u l=180n
M556 t219 nq4 0 0 nch w=1u l=180n
M557 t217 nw54 vdd vdd pch w=2u l=180n
M558 t217 t216 vdd vdd pch w=2u l=180n
CT220 t220 0 0.1f
M559 t217 nw54 t220 0 nch w=1u l=180n
M560 t220 t216 0 0 nch w=1u l=180n
M561 t218 nq4 vdd vdd pch w=2u l=180n
M562 t218 t216 vdd vdd pch w=2u l=180n
CT221 t221 0 0.1f
M563 t218 nq4 t221 0 nch w=1u l=180n
M564 t221 t216 0 0 nch w=1u l=180n
M565 nw62 t217 vdd vdd pch w=2u l=180n
M566 nw62 t218 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M567 nw62 t217 t222 0 nch w=1u l=180n
M568 t222 t218 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
M569 nw63 nw58 vdd vdd pch w=2u l=180n
M570 nw63 nq9 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M571 nw63 nw58 t223 0 nch w=1u l=180n
M572 t223 nq9 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
M573 nw64 nw62 0 0 nch w=1u l=180n
M574 nw64 nq14 0 0 nch w=1u l=180n
CT224 t224 0 0.1f
M575 t224 nw62 vdd vdd pch w=2u l=180n
M576 nw64 nq14 t224 vdd pch w=2u l=180n
Cnw64 nw64 0 2f
CT225 t225 0 0.1f
M577 t225 nq1 vdd vdd pch w=2u l=180n
M578 t225 ni3 vdd vdd pch w=2u l=180n
CT226 t226 0 0.1f
M579 t225 nq1 t226 0 nch w=1u l=180n
M580 t226 ni3 0 0 nch w=1u l=180n
M581 nw65 t225 vdd vdd pch w=2u l=180n
M582 nw65 t225 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
CT227 t227 0 0.1f
M583 t227 nq4 0 0 nch w=1u l=180n
M584 t227 nw33 0 0 nch w=1u l=180n
CT228 t228 0 0.1f
M585 t228 nq4 vdd vdd pch w=2u l=180n
M586 t227 nw33 t228 vdd pch w=2u l=180n
M587 nw66 t227 vdd vdd pch w=2u l=180n
M588 nw66 t227 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
CT229 t229 0 0.1f
CT230 t230 0 0.1f
CT231 t231 0 0.1f
M589 t229 nq7 vdd vdd pch w=2u l=180n
M590 t229 nw38 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M591 t229 nq7 t232 0 nch w=1u l=180n
M592 t232 nw38 0 0 nch w=1u l=180n
M593 t230 nq7 vdd vdd pch w=2u l=180n
M594 t230 t229 vdd vdd pch w=2u l=180n
CT233 t233 0 0.1f
M595 t230 nq7 t233 0 nch w=1u l=180n
M596 t233 t229 0 0 nch w=1u l=180n
M597 t231 nw38 vdd vdd pch w=2u l=180n
M598 t231 t229 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M599 t231 nw38 t234 0 nch w=1u l=180n
M600 t234 t229 0 0 nch w=1u l=180n
M601 nw67 t230 vdd vdd pch w=2u l=180n
M602 nw67 t231 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M603 nw67 t230 t235 0 nch w=1u l=180n
M604 t235 t231 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
M605 nw68 nq10 vdd vdd pch w=2u l=180n
M606 nw68 nw43 vdd vdd pch w=2u l=180n
CT236 t236 0 0.1f
M607 nw68 nq10 t236 0 nch w=1u l=180n
M608 t236 nw43 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
M609 nw69 nq13 0 0 nch w=1u l=180n
M610 nw69 nw48 0 0 nch w=1u l=180n
CT237 t237 0 0.1f
M611 t237 nq13 vdd vdd pch w=2u l=180n
M612 nw69 nw48 t237 vdd pch w=2u l=180n
Cnw69 nw69 0 2f
CT238 t238 0 0.1f
M613 t238 ni0 vdd vdd pch w=2u l=180n
M614 t238 nw53 vdd vdd pch w=2u l=180n
CT239 t239 0 0.1f
M615 t238 ni0 t239 0 nch w=1u l=180n
M616 t239 nw53 0 0 nch w=1u l=180n
M617 nw70 t238 vdd vdd pch w=2u l=180n
M618 nw70 t238 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
CT240 t240 0 0.1f
M619 t240 ni3 0 0 nch w=1u l=180n
M620 t240 nw58 0 0 nch w=1u l=180n
CT241 t241 0 0.1f
M621 t241 ni3 vdd vdd pch w=2u l=180n
M622 t240 nw58 t241 vdd pch w=2u l=180n
M623 nw71 t240 vdd vdd pch w=2u l=180n
M624 nw71 t240 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
CT242 t242 0 0.1f
CT243 t243 0 0.1f
CT244 t244 0 0.1f
M625 t242 ni6 vdd vdd pch w=2u l=180n
M626 t242 nw63 vdd vdd pch w=2u l=180n
CT245 t245 0 0.1f
M627 t242 ni6 t245 0 nch w=1u l=180n
M628 t245 nw63 0 0 nch w=1u l=180n
M629 t243 ni6 vdd vdd pch w=2u l=180n
M630 t243 t242 vdd vdd pch w=2u l=180n
CT246 t246 0 0.1f
M631 t243 ni6 t246 0 nch w=1u l=180n
M632 t246 t242 0 0 nch w=1u l=180n
M633 t244 nw63 vdd vdd pch w=2u l=180n
M634 t244 t242 vdd vdd pch w=2u l=180n
CT247 t247 0 0.1f
M635 t244 nw63 t247 0 nch w=1u l=180n
M636 t247 t242 0 0 nch w=1u l=180n
M637 nw72 t243 vdd vdd pch w=2u l=180n
M638 nw72 t244 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M639 nw72 t243 t248 0 nch w=1u l=180n
M640 t248 t244 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M641 nw73 nw34 vdd vdd pch w=2u l=180n
M642 nw73 nw68 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M643 nw73 nw34 t249 0 nch w=1u l=180n
M644 t249 nw68 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
M645 nw74 nw37 0 0 nch w=1u l=180n
M646 nw74 nw73 0 0 nch w=1u l=180n
CT250 t250 0 0.1f
M647 t250 nw37 vdd vdd pch w=2u l=180n
M648 nw74 nw73 t250 vdd pch w=2u l=180n
Cnw74 nw74 0 2f
CT251 t251 0 0.1f
M649 t251 nw40 vdd vdd pch w=2u l=180n
M650 t251 nq3 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M651 t251 nw40 t252 0 nch w=1u l=180n
M652 t252 nq3 0 0 nch w=1u l=180n
M653 nw75 t251 vdd vdd pch w=2u l=180n
M654 nw75 t251 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
CT253 t253 0 0.1f
M655 t253 nw43 0 0 nch w=1u l=180n
M656 t253 nq7 0 0 nch w=1u l=180n
CT254 t254 0 0.1f
M657 t254 nw43 vdd vdd pch w=2u l=180n
M658 t253 nq7 t254 vdd pch w=2u l=180n
M659 nw76 t253 vdd vdd pch w=2u l=180n
M660 nw76 t253 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
CT255 t255 0 0.1f
CT256 t256 0 0.1f
CT257 t257 0 0.1f
M661 t255 nw46 vdd vdd pch w=2u l=180n
M662 t255 nq11 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M663 t255 nw46 t258 0 nch w=1u l=180n
M664 t258 nq11 0 0 nch w=1u l=180n
M665 t256 nw46 vdd vdd pch w=2u l=180n
M666 t256 t255 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M667 t256 nw46 t259 0 nch w=1u l=180n
M668 t259 t255 0 0 nch w=1u l=180n
M669 t257 nq11 vdd vdd pch w=2u l=180n
M670 t257 t255 vdd vdd pch w=2u l=180n
CT260 t260 0 0.1f
M671 t257 nq11 t260 0 nch w=1u l=180n
M672 t260 t255 0 0 nch w=1u l=180n
M673 nw77 t256 vdd vdd pch w=2u l=180n
M674 nw77 t257 vdd vdd pch w=2u l=180n
CT261 t261 0 0.1f
M675 nw77 t256 t261 0 nch w=1u l=180n
M676 t261 t257 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
M677 nw78 nw49 vdd vdd pch w=2u l=180n
M678 nw78 nq15 vdd vdd pch w=2u l=180n
CT262 t262 0 0.1f
M679 nw78 nw49 t262 0 nch w=1u l=180n
M680 t262 nq15 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M681 nw79 nw52 0 0 nch w=1u l=180n
M682 nw79 ni3 0 0 nch w=1u l=180n
CT263 t263 0 0.1f
M683 t263 nw52 vdd vdd pch w=2u l=180n
M684 nw79 ni3 t263 vdd pch w=2u l=180n
Cnw79 nw79 0 2f
CT264 t264 0 0.1f
M685 t264 nw55 vdd vdd pch w=2u l=180n
M686 t264 ni7 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M687 t264 nw55 t265 0 nch w=1u l=180n
M688 t265 ni7 0 0 nch w=1u l=180n
M689 nw80 t264 vdd vdd pch w=2u l=180n
M690 nw80 t264 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
CT266 t266 0 0.1f
M691 t266 nw58 0 0 nch w=1u l=180n
M692 t266 nw36 0 0 nch w=1u l=180n
CT267 t267 0 0.1f
M693 t267 nw58 vdd vdd pch w=2u l=180n
M694 t266 nw36 t267 vdd pch w=2u l=180n
M695 nw81 t266 vdd vdd pch w=2u l=180n
M696 nw81 t266 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
CT268 t268 0 0.1f
CT269 t269 0 0.1f
CT270 t270 0 0.1f
M697 t268 nw61 vdd vdd pch w=2u l=180n
M698 t268 nw40 vdd vdd pch w=2u l=180n
CT271 t271 0 0.1f
M699 t268 nw61 t271 0 nch w=1u l=180n
M700 t271 nw40 0 0 nch w=1u l=180n
M701 t269 nw61 vdd vdd pch w=2u l=180n
M702 t269 t268 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M703 t269 nw61 t272 0 nch w=1u l=180n
M704 t272 t268 0 0 nch w=1u l=180n
M705 t270 nw40 vdd vdd pch w=2u l=180n
M706 t270 t268 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M707 t270 nw40 t273 0 nch w=1u l=180n
M708 t273 t268 0 0 nch w=1u l=180n
M709 nw82 t269 vdd vdd pch w=2u l=180n
M710 nw82 t270 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M711 nw82 t269 t274 0 nch w=1u l=180n
M712 t274 t270 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
M713 nw83 nw64 vdd vdd pch w=2u l=180n
M714 nw83 nw44 vdd vdd pch w=2u l=180n
CT275 t275 0 0.1f
M715 nw83 nw64 t275 0 nch w=1u l=180n
M716 t275 nw44 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
M717 nw84 nw67 0 0 nch w=1u l=180n
M718 nw84 nw48 0 0 nch w=1u l=180n
CT276 t276 0 0.1f
M719 t276 nw67 vdd vdd pch w=2u l=180n
M720 nw84 nw48 t276 vdd pch w=2u l=180n
Cnw84 nw84 0 2f
CT277 t277 0 0.1f
M721 t277 nw70 vdd vdd pch w=2u l=180n
M722 t277 nw52 vdd vdd pch w=2u l=180n
CT278 t278 0 0.1f
M723 t277 nw70 t278 0 nch w=1u l=180n
M724 t278 nw52 0 0 nch w=1u l=180n
M725 nw85 t277 vdd vdd pch w=2u l=180n
M726 nw85 t277 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
CT279 t279 0 0.1f
M727 t279 nw73 0 0 nch w=1u l=180n
M728 t279 nw56 0 0 nch w=1u l=180n
CT280 t280 0 0.1f
M729 t280 nw73 vdd vdd pch w=2u l=180n
M730 t279 nw56 t280 vdd pch w=2u l=180n
M731 nw86 t279 vdd vdd pch w=2u l=180n
M732 nw86 t279 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
CT281 t281 0 0.1f
CT282 t282 0 0.1f
CT283 t283 0 0.1f
M733 t281 nw76 vdd vdd pch w=2u l=180n
M734 t281 nw60 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M735 t281 nw76 t284 0 nch w=1u l=180n
M736 t284 nw60 0 0 nch w=1u l=180n
M737 t282 nw76 vdd vdd pch w=2u l=180n
M738 t282 t281 vdd vdd pch w=2u l=180n
CT285 t285 0 0.1f
M739 t282 nw76 t285 0 nch w=1u l=180n
M740 t285 t281 0 0 nch w=1u l=180n
M741 t283 nw60 vdd vdd pch w=2u l=180n
M742 t283 t281 vdd vdd pch w=2u l=180n
CT286 t286 0 0.1f
M743 t283 nw60 t286 0 nch w=1u l=180n
M744 t286 t281 0 0 nch w=1u l=180n
M745 nw87 t282 vdd vdd pch w=2u l=180n
M746 nw87 t283 vdd vdd pch w=2u l=180n
CT287 t287 0 0.1f
M747 nw87 t282 t287 0 nch w=1u l=180n
M748 t287 t283 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M749 nw88 nw79 vdd vdd pch w=2u l=180n
M750 nw88 nw64 vdd vdd pch w=2u l=180n
CT288 t288 0 0.1f
M751 nw88 nw79 t288 0 nch w=1u l=180n
M752 t288 nw64 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
M753 nw89 nw82 0 0 nch w=1u l=180n
M754 nw89 nw68 0 0 nch w=1u l=180n
CT289 t289 0 0.1f
M755 t289 nw82 vdd vdd pch w=2u l=180n
M756 nw89 nw68 t289 vdd pch w=2u l=180n
Cnw89 nw89 0 2f
CT290 t290 0 0.1f
M757 t290 nw85 vdd vdd pch w=2u l=180n
M758 t290 nw72 vdd vdd pch w=2u l=180n
CT291 t291 0 0.1f
M759 t290 nw85 t291 0 nch w=1u l=180n
M760 t291 nw72 0 0 nch w=1u l=180n
M761 nw90 t290 vdd vdd pch w=2u l=180n
M762 nw90 t290 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
CT292 t292 0 0.1f
M763 t292 nw88 0 0 nch w=1u l=180n
M764 t292 nw76 0 0 nch w=1u l=180n
CT293 t293 0 0.1f
M765 t293 nw88 vdd vdd pch w=2u l=180n
M766 t292 nw76 t293 vdd pch w=2u l=180n
M767 nw91 t292 vdd vdd pch w=2u l=180n
M768 nw91 t292 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
CT294 t294 0 0.1f
CT295 t295 0 0.1f
CT296 t296 0 0.1f
M769 t294 nw91 vdd vdd pch w=2u l=180n
M770 t294 nw80 vdd vdd pch w=2u l=180n
CT297 t297 0 0.1f
M771 t294 nw91 t297 0 nch w=1u l=180n
M772 t297 nw80 0 0 nch w=1u l=180n
M773 t295 nw91 vdd vdd pch w=2u l=180n
M774 t295 t294 vdd vdd pch w=2u l=180n
CT298 t298 0 0.1f
M775 t295 nw91 t298 0 nch w=1u l=180n
M776 t298 t294 0 0 nch w=1u l=180n
M777 t296 nw80 vdd vdd pch w=2u l=180n
M778 t296 t294 vdd vdd pch w=2u l=180n
CT299 t299 0 0.1f
M779 t296 nw80 t299 0 nch w=1u l=180n
M780 t299 t294 0 0 nch w=1u l=180n
M781 nw92 t295 vdd vdd pch w=2u l=180n
M782 nw92 t296 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M783 nw92 t295 t300 0 nch w=1u l=180n
M784 t300 t296 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M785 nw93 nq1 vdd vdd pch w=2u l=180n
M786 nw93 nw84 vdd vdd pch w=2u l=180n
CT301 t301 0 0.1f
M787 nw93 nq1 t301 0 nch w=1u l=180n
M788 t301 nw84 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M789 nw94 nq3 0 0 nch w=1u l=180n
M790 nw94 nw88 0 0 nch w=1u l=180n
CT302 t302 0 0.1f
M791 t302 nq3 vdd vdd pch w=2u l=180n
M792 nw94 nw88 t302 vdd pch w=2u l=180n
Cnw94 nw94 0 2f
CT303 t303 0 0.1f
M793 t303 nq5 vdd vdd pch w=2u l=180n
M794 t303 nw92 vdd vdd pch w=2u l=180n
CT304 t304 0 0.1f
M795 t303 nq5 t304 0 nch w=1u l=180n
M796 t304 nw92 0 0 nch w=1u l=180n
M797 nw95 t303 vdd vdd pch w=2u l=180n
M798 nw95 t303 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
CT305 t305 0 0.1f
M799 t305 nq7 0 0 nch w=1u l=180n
M800 t305 nq0 0 0 nch w=1u l=180n
CT306 t306 0 0.1f
M801 t306 nq7 vdd vdd pch w=2u l=180n
M802 t305 nq0 t306 vdd pch w=2u l=180n
M803 nw96 t305 vdd vdd pch w=2u l=180n
M804 nw96 t305 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
CT307 t307 0 0.1f
CT308 t308 0 0.1f
CT309 t309 0 0.1f
M805 t307 nq9 vdd vdd pch w=2u l=180n
M806 t307 nq3 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M807 t307 nq9 t310 0 nch w=1u l=180n
M808 t310 nq3 0 0 nch w=1u l=180n
M809 t308 nq9 vdd vdd pch w=2u l=180n
M810 t308 t307 vdd vdd pch w=2u l=180n
CT311 t311 0 0.1f
M811 t308 nq9 t311 0 nch w=1u l=180n
M812 t311 t307 0 0 nch w=1u l=180n
M813 t309 nq3 vdd vdd pch w=2u l=180n
M814 t309 t307 vdd vdd pch w=2u l=180n
CT312 t312 0 0.1f
M815 t309 nq3 t312 0 nch w=1u l=180n
M816 t312 t307 0 0 nch w=1u l=180n
M817 nw97 t308 vdd vdd pch w=2u l=180n
M818 nw97 t309 vdd vdd pch w=2u l=180n
CT313 t313 0 0.1f
M819 nw97 t308 t313 0 nch w=1u l=180n
M820 t313 t309 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
M821 nw98 nq11 vdd vdd pch w=2u l=180n
M822 nw98 nq6 vdd vdd pch w=2u l=180n
CT314 t314 0 0.1f
M823 nw98 nq11 t314 0 nch w=1u l=180n
M824 t314 nq6 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
M825 nw99 nq13 0 0 nch w=1u l=180n
M826 nw99 nq9 0 0 nch w=1u l=180n
CT315 t315 0 0.1f
M827 t315 nq13 vdd vdd pch w=2u l=180n
M828 nw99 nq9 t315 vdd pch w=2u l=180n
Cnw99 nw99 0 2f
CT316 t316 0 0.1f
M829 t316 nq15 vdd vdd pch w=2u l=180n
M830 t316 nq12 vdd vdd pch w=2u l=180n
CT317 t317 0 0.1f
M831 t316 nq15 t317 0 nch w=1u l=180n
M832 t317 nq12 0 0 nch w=1u l=180n
M833 nw100 t316 vdd vdd pch w=2u l=180n
M834 nw100 t316 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
CT318 t318 0 0.1f
M835 t318 ni1 0 0 nch w=1u l=180n
M836 t318 nq15 0 0 nch w=1u l=180n
CT319 t319 0 0.1f
M837 t319 ni1 vdd vdd pch w=2u l=180n
M838 t318 nq15 t319 vdd pch w=2u l=180n
M839 nw101 t318 vdd vdd pch w=2u l=180n
M840 nw101 t318 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
CT320 t320 0 0.1f
CT321 t321 0 0.1f
CT322 t322 0 0.1f
M841 t320 ni3 vdd vdd pch w=2u l=180n
M842 t320 ni2 vdd vdd pch w=2u l=180n
CT323 t323 0 0.1f
M843 t320 ni3 t323 0 nch w=1u l=180n
M844 t323 ni2 0 0 nch w=1u l=180n
M845 t321 ni3 vdd vdd pch w=2u l=180n
M846 t321 t320 vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M847 t321 ni3 t324 0 nch w=1u l=180n
M848 t324 t320 0 0 nch w=1u l=180n
M849 t322 ni2 vdd vdd pch w=2u l=180n
M850 t322 t320 vdd vdd pch w=2u l=180n
CT325 t325 0 0.1f
M851 t322 ni2 t325 0 nch w=1u l=180n
M852 t325 t320 0 0 nch w=1u l=180n
M853 nw102 t321 vdd vdd pch w=2u l=180n
M854 nw102 t322 vdd vdd pch w=2u l=180n
CT326 t326 0 0.1f
M855 nw102 t321 t326 0 nch w=1u l=180n
M856 t326 t322 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
M857 nw103 ni5 vdd vdd pch w=2u l=180n
M858 nw103 nw78 vdd vdd pch w=2u l=180n
CT327 t327 0 0.1f
M859 nw103 ni5 t327 0 nch w=1u l=180n
M860 t327 nw78 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
M861 nw104 ni7 0 0 nch w=1u l=180n
M862 nw104 nw33 0 0 nch w=1u l=180n
CT328 t328 0 0.1f
M863 t328 ni7 vdd vdd pch w=2u l=180n
M864 nw104 nw33 t328 vdd pch w=2u l=180n
Cnw104 nw104 0 2f
CT329 t329 0 0.1f
M865 t329 nw34 vdd vdd pch w=2u l=180n
M866 t329 nw36 vdd vdd pch w=2u l=180n
CT330 t330 0 0.1f
M867 t329 nw34 t330 0 nch w=1u l=180n
M868 t330 nw36 0 0 nch w=1u l=180n
M869 nw105 t329 vdd vdd pch w=2u l=180n
M870 nw105 t329 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
CT331 t331 0 0.1f
M871 t331 nw36 0 0 nch w=1u l=180n
M872 t331 nw39 0 0 nch w=1u l=180n
CT332 t332 0 0.1f
M873 t332 nw36 vdd vdd pch w=2u l=180n
M874 t331 nw39 t332 vdd pch w=2u l=180n
M875 nw106 t331 vdd vdd pch w=2u l=180n
M876 nw106 t331 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
CT333 t333 0 0.1f
CT334 t334 0 0.1f
CT335 t335 0 0.1f
M877 t333 nw38 vdd vdd pch w=2u l=180n
M878 t333 nw42 vdd vdd pch w=2u l=180n
CT336 t336 0 0.1f
M879 t333 nw38 t336 0 nch w=1u l=180n
M880 t336 nw42 0 0 nch w=1u l=180n
M881 t334 nw38 vdd vdd pch w=2u l=180n
M882 t334 t333 vdd vdd pch w=2u l=180n
CT337 t337 0 0.1f
M883 t334 nw38 t337 0 nch w=1u l=180n
M884 t337 t333 0 0 nch w=1u l=180n
M885 t335 nw42 vdd vdd pch w=2u l=180n
M886 t335 t333 vdd vdd pch w=2u l=180n
CT338 t338 0 0.1f
M887 t335 nw42 t338 0 nch w=1u l=180n
M888 t338 t333 0 0 nch w=1u l=180n
M889 nw107 t334 vdd vdd pch w=2u l=180n
M890 nw107 t335 vdd vdd pch w=2u l=180n
CT339 t339 0 0.1f
M891 nw107 t334 t339 0 nch w=1u l=180n
M892 t339 t335 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
M893 nw108 nw40 vdd vdd pch w=2u l=180n
M894 nw108 nw45 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M895 nw108 nw40 t340 0 nch w=1u l=180n
M896 t340 nw45 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
M897 nw109 nw42 0 0 nch w=1u l=180n
M898 nw109 nw48 0 0 nch w=1u l=180n
CT341 t341 0 0.1f
M899 t341 nw42 vdd vdd pch w=2u l=180n
M900 nw109 nw48 t341 vdd pch w=2u l=180n
Cnw109 nw109 0 2f
CT342 t342 0 0.1f
M901 t342 nw44 vdd vdd pch w=2u l=180n
M902 t342 nw51 vdd vdd pch w=2u l=180n
CT343 t343 0 0.1f
M903 t342 nw44 t343 0 nch w=1u l=180n
M904 t343 nw51 0 0 nch w=1u l=180n
M905 nw110 t342 vdd vdd pch w=2u l=180n
M906 nw110 t342 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
CT344 t344 0 0.1f
M907 t344 nw46 0 0 nch w=1u l=180n
M908 t344 nw54 0 0 nch w=1u l=180n
CT345 t345 0 0.1f
M909 t345 nw46 vdd vdd pch w=2u l=180n
M910 t344 nw54 t345 vdd pch w=2u l=180n
M911 nw111 t344 vdd vdd pch w=2u l=180n
M912 nw111 t344 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
CT346 t346 0 0.1f
CT347 t347 0 0.1f
CT348 t348 0 0.1f
M913 t346 nw48 vdd vdd pch w=2u l=180n
M914 t346 nw57 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M915 t346 nw48 t349 0 nch w=1u l=180n
M916 t349 nw57 0 0 nch w=1u l=180n
M917 t347 nw48 vdd vdd pch w=2u l=180n
M918 t347 t346 vdd vdd pch w=2u l=180n
CT350 t350 0 0.1f
M919 t347 nw48 t350 0 nch w=1u l=180n
M920 t350 t346 0 0 nch w=1u l=180n
M921 t348 nw57 vdd vdd pch w=2u l=180n
M922 t348 t346 vdd vdd pch w=2u l=180n
CT351 t351 0 0.1f
M923 t348 nw57 t351 0 nch w=1u l=180n
M924 t351 t346 0 0 nch w=1u l=180n
M925 nw112 t347 vdd vdd pch w=2u l=180n
M926 nw112 t348 vdd vdd pch w=2u l=180n
CT352 t352 0 0.1f
M927 nw112 t347 t352 0 nch w=1u l=180n
M928 t352 t348 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
M929 nw113 nw50 vdd vdd pch w=2u l=180n
M930 nw113 nw60 vdd vdd pch w=2u l=180n
CT353 t353 0 0.1f
M931 nw113 nw50 t353 0 nch w=1u l=180n
M932 t353 nw60 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
M933 nw114 nw52 0 0 nch w=1u l=180n
M934 nw114 nw63 0 0 nch w=1u l=180n
CT354 t354 0 0.1f
M935 t354 nw52 vdd vdd pch w=2u l=180n
M936 nw114 nw63 t354 vdd pch w=2u l=180n
Cnw114 nw114 0 2f
CT355 t355 0 0.1f
M937 t355 nw54 vdd vdd pch w=2u l=180n
M938 t355 nw66 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M939 t355 nw54 t356 0 nch w=1u l=180n
M940 t356 nw66 0 0 nch w=1u l=180n
M941 nw115 t355 vdd vdd pch w=2u l=180n
M942 nw115 t355 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
CT357 t357 0 0.1f
M943 t357 nw56 0 0 nch w=1u l=180n
M944 t357 nw69 0 0 nch w=1u l=180n
CT358 t358 0 0.1f
M945 t358 nw56 vdd vdd pch w=2u l=180n
M946 t357 nw69 t358 vdd pch w=2u l=180n
M947 nw116 t357 vdd vdd pch w=2u l=180n
M948 nw116 t357 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
CT359 t359 0 0.1f
CT360 t360 0 0.1f
CT361 t361 0 0.1f
M949 t359 nw58 vdd vdd pch w=2u l=180n
M950 t359 nw72 vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M951 t359 nw58 t362 0 nch w=1u l=180n
M952 t362 nw72 0 0 nch w=1u l=180n
M953 t360 nw58 vdd vdd pch w=2u l=180n
M954 t360 t359 vdd vdd pch w=2u l=180n
CT363 t363 0 0.1f
M955 t360 nw58 t363 0 nch w=1u l=180n
M956 t363 t359 0 0 nch w=1u l=180n
M957 t361 nw72 vdd vdd pch w=2u l=180n
M958 t361 t359 vdd vdd pch w=2u l=180n
CT364 t364 0 0.1f
M959 t361 nw72 t364 0 nch w=1u l=180n
M960 t364 t359 0 0 nch w=1u l=180n
M961 nw117 t360 vdd vdd pch w=2u l=180n
M962 nw117 t361 vdd vdd pch w=2u l=180n
CT365 t365 0 0.1f
M963 nw117 t360 t365 0 nch w=1u l=180n
M964 t365 t361 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
M965 nw118 nw60 vdd vdd pch w=2u l=180n
M966 nw118 nw75 vdd vdd pch w=2u l=180n
CT366 t366 0 0.1f
M967 nw118 nw60 t366 0 nch w=1u l=180n
M968 t366 nw75 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
M969 nw119 nw62 0 0 nch w=1u l=180n
M970 nw119 nw78 0 0 nch w=1u l=180n
CT367 t367 0 0.1f
M971 t367 nw62 vdd vdd pch w=2u l=180n
M972 nw119 nw78 t367 vdd pch w=2u l=180n
Cnw119 nw119 0 2f
CT368 t368 0 0.1f
M973 t368 nw64 vdd vdd pch w=2u l=180n
M974 t368 nw81 vdd vdd pch w=2u l=180n
CT369 t369 0 0.1f
M975 t368 nw64 t369 0 nch w=1u l=180n
M976 t369 nw81 0 0 nch w=1u l=180n
M977 nw120 t368 vdd vdd pch w=2u l=180n
M978 nw120 t368 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
CT370 t370 0 0.1f
M979 t370 nw66 0 0 nch w=1u l=180n
M980 t370 nw84 0 0 nch w=1u l=180n
CT371 t371 0 0.1f
M981 t371 nw66 vdd vdd pch w=2u l=180n
M982 t370 nw84 t371 vdd pch w=2u l=180n
M983 nw121 t370 vdd vdd pch w=2u l=180n
M984 nw121 t370 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
CT372 t372 0 0.1f
CT373 t373 0 0.1f
CT374 t374 0 0.1f
M985 t372 nw68 vdd vdd pch w=2u l=180n
M986 t372 nw87 vdd vdd pch w=2u l=180n
CT375 t375 0 0.1f
M987 t372 nw68 t375 0 nch w=1u l=180n
M988 t375 nw87 0 0 nch w=1u l=180n
M989 t373 nw68 vdd vdd pch w=2u l=180n
M990 t373 t372 vdd vdd pch w=2u l=180n
CT376 t376 0 0.1f
M991 t373 nw68 t376 0 nch w=1u l=180n
M992 t376 t372 0 0 nch w=1u l=180n
M993 t374 nw87 vdd vdd pch w=2u l=180n
M994 t374 t372 vdd vdd pch w=2u l=180n
CT377 t377 0 0.1f
M995 t374 nw87 t377 0 nch w=1u l=180n
M996 t377 t372 0 0 nch w=1u l=180n
M997 nw122 t373 vdd vdd pch w=2u l=180n
M998 nw122 t374 vdd vdd pch w=2u l=180n
CT378 t378 0 0.1f
M999 nw122 t373 t378 0 nch w=1u l=180n
M1000 t378 t374 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
M1001 nw123 nw70 vdd vdd pch w=2u l=180n
M1002 nw123 nw90 vdd vdd pch w=2u l=180n
CT379 t379 0 0.1f
M1003 nw123 nw70 t379 0 nch w=1u l=180n
M1004 t379 nw90 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
M1005 nw124 nw72 0 0 nch w=1u l=180n
M1006 nw124 nw93 0 0 nch w=1u l=180n
CT380 t380 0 0.1f
M1007 t380 nw72 vdd vdd pch w=2u l=180n
M1008 nw124 nw93 t380 vdd pch w=2u l=180n
Cnw124 nw124 0 2f
CT381 t381 0 0.1f
M1009 t381 nw74 vdd vdd pch w=2u l=180n
M1010 t381 nw96 vdd vdd pch w=2u l=180n
CT382 t382 0 0.1f
M1011 t381 nw74 t382 0 nch w=1u l=180n
M1012 t382 nw96 0 0 nch w=1u l=180n
M1013 nw125 t381 vdd vdd pch w=2u l=180n
M1014 nw125 t381 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
CT383 t383 0 0.1f
M1015 t383 nw76 0 0 nch w=1u l=180n
M1016 t383 nw99 0 0 nch w=1u l=180n
CT384 t384 0 0.1f
M1017 t384 nw76 vdd vdd pch w=2u l=180n
M1018 t383 nw99 t384 vdd pch w=2u l=180n
M1019 nw126 t383 vdd vdd pch w=2u l=180n
M1020 nw126 t383 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
CT385 t385 0 0.1f
CT386 t386 0 0.1f
CT387 t387 0 0.1f
M1021 t385 nw78 vdd vdd pch w=2u l=180n
M1022 t385 nw102 vdd vdd pch w=2u l=180n
CT388 t388 0 0.1f
M1023 t385 nw78 t388 0 nch w=1u l=180n
M1024 t388 nw102 0 0 nch w=1u l=180n
M1025 t386 nw78 vdd vdd pch w=2u l=180n
M1026 t386 t385 vdd vdd pch w=2u l=180n
CT389 t389 0 0.1f
M1027 t386 nw78 t389 0 nch w=1u l=180n
M1028 t389 t385 0 0 nch w=1u l=180n
M1029 t387 nw102 vdd vdd pch w=2u l=180n
M1030 t387 t385 vdd vdd pch w=2u l=180n
CT390 t390 0 0.1f
M1031 t387 nw102 t390 0 nch w=1u l=180n
M1032 t390 t385 0 0 nch w=1u l=180n
M1033 nw127 t386 vdd vdd pch w=2u l=180n
M1034 nw127 t387 vdd vdd pch w=2u l=180n
CT391 t391 0 0.1f
M1035 nw127 t386 t391 0 nch w=1u l=180n
M1036 t391 t387 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
M1037 nw128 nw80 vdd vdd pch w=2u l=180n
M1038 nw128 nw105 vdd vdd pch w=2u l=180n
CT392 t392 0 0.1f
M1039 nw128 nw80 t392 0 nch w=1u l=180n
M1040 t392 nw105 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
M1041 nw129 nw82 0 0 nch w=1u l=180n
M1042 nw129 nw108 0 0 nch w=1u l=180n
CT393 t393 0 0.1f
M1043 t393 nw82 vdd vdd pch w=2u l=180n
M1044 nw129 nw108 t393 vdd pch w=2u l=180n
Cnw129 nw129 0 2f
CT394 t394 0 0.1f
M1045 t394 nw84 vdd vdd pch w=2u l=180n
M1046 t394 nw111 vdd vdd pch w=2u l=180n
CT395 t395 0 0.1f
M1047 t394 nw84 t395 0 nch w=1u l=180n
M1048 t395 nw111 0 0 nch w=1u l=180n
M1049 nw130 t394 vdd vdd pch w=2u l=180n
M1050 nw130 t394 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
CT396 t396 0 0.1f
M1051 t396 nw86 0 0 nch w=1u l=180n
M1052 t396 nw114 0 0 nch w=1u l=180n
CT397 t397 0 0.1f
M1053 t397 nw86 vdd vdd pch w=2u l=180n
M1054 t396 nw114 t397 vdd pch w=2u l=180n
M1055 nw131 t396 vdd vdd pch w=2u l=180n
M1056 nw131 t396 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
CT398 t398 0 0.1f
CT399 t399 0 0.1f
CT400 t400 0 0.1f
M1057 t398 nw88 vdd vdd pch w=2u l=180n
M1058 t398 nw117 vdd vdd pch w=2u l=180n
CT401 t401 0 0.1f
M1059 t398 nw88 t401 0 nch w=1u l=180n
M1060 t401 nw117 0 0 nch w=1u l=180n
M1061 t399 nw88 vdd vdd pch w=2u l=180n
M1062 t399 t398 vdd vdd pch w=2u l=180n
CT402 t402 0 0.1f
M1063 t399 nw88 t402 0 nch w=1u l=180n
M1064 t402 t398 0 0 nch w=1u l=180n
M1065 t400 nw117 vdd vdd pch w=2u l=180n
M1066 t400 t398 vdd vdd pch w=2u l=180n
CT403 t403 0 0.1f
M1067 t400 nw117 t403 0 nch w=1u l=180n
M1068 t403 t398 0 0 nch w=1u l=180n
M1069 nw132 t399 vdd vdd pch w=2u l=180n
M1070 nw132 t400 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M1071 nw132 t399 t404 0 nch w=1u l=180n
M1072 t404 t400 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
M1073 nw133 nw90 vdd vdd pch w=2u l=180n
M1074 nw133 nw120 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M1075 nw133 nw90 t405 0 nch w=1u l=180n
M1076 t405 nw120 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
M1077 nw134 nw92 0 0 nch w=1u l=180n
M1078 nw134 nw123 0 0 nch w=1u l=180n
CT406 t406 0 0.1f
M1079 t406 nw92 vdd vdd pch w=2u l=180n
M1080 nw134 nw123 t406 vdd pch w=2u l=180n
Cnw134 nw134 0 2f
CT407 t407 0 0.1f
M1081 t407 nw94 vdd vdd pch w=2u l=180n
M1082 t407 nw126 vdd vdd pch w=2u l=180n
CT408 t408 0 0.1f
M1083 t407 nw94 t408 0 nch w=1u l=180n
M1084 t408 nw126 0 0 nch w=1u l=180n
M1085 nw135 t407 vdd vdd pch w=2u l=180n
M1086 nw135 t407 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
CT409 t409 0 0.1f
M1087 t409 nw96 0 0 nch w=1u l=180n
M1088 t409 nw129 0 0 nch w=1u l=180n
CT410 t410 0 0.1f
M1089 t410 nw96 vdd vdd pch w=2u l=180n
M1090 t409 nw129 t410 vdd pch w=2u l=180n
M1091 nw136 t409 vdd vdd pch w=2u l=180n
M1092 nw136 t409 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
CT411 t411 0 0.1f
CT412 t412 0 0.1f
CT413 t413 0 0.1f
M1093 t411 nw98 vdd vdd pch w=2u l=180n
M1094 t411 nw132 vdd vdd pch w=2u l=180n
CT414 t414 0 0.1f
M1095 t411 nw98 t414 0 nch w=1u l=180n
M1096 t414 nw132 0 0 nch w=1u l=180n
M1097 t412 nw98 vdd vdd pch w=2u l=180n
M1098 t412 t411 vdd vdd pch w=2u l=180n
CT415 t415 0 0.1f
M1099 t412 nw98 t415 0 nch w=1u l=180n
M1100 t415 t411 0 0 nch w=1u l=180n
M1101 t413 nw132 vdd vdd pch w=2u l=180n
M1102 t413 t411 vdd vdd pch w=2u l=180n
CT416 t416 0 0.1f
M1103 t413 nw132 t416 0 nch w=1u l=180n
M1104 t416 t411 0 0 nch w=1u l=180n
M1105 nw137 t412 vdd vdd pch w=2u l=180n
M1106 nw137 t413 vdd vdd pch w=2u l=180n
CT417 t417 0 0.1f
M1107 nw137 t412 t417 0 nch w=1u l=180n
M1108 t417 t413 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
M1109 nw138 nw100 vdd vdd pch w=2u l=180n
M1110 nw138 nw135 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M1111 nw138 nw100 t418 0 nch w=1u l=180n
M1112 t418 nw135 0 0 nch w=1u l=180n
Cnw138 nw138 0 2f
M1113 nw139 nw102 0 0 nch w=1u l=180n
M1114 nw139 nw138 0 0 nch w=1u l=180n
CT419 t419 0 0.1f
M1115 t419 nw102 vdd vdd pch w=2u l=180n
M1116 nw139 nw138 t419 vdd pch w=2u l=180n
Cnw139 nw139 0 2f
CT420 t420 0 0.1f
M1117 t420 nw104 vdd vdd pch w=2u l=180n
M1118 t420 nq1 vdd vdd pch w=2u l=180n
CT421 t421 0 0.1f
M1119 t420 nw104 t421 0 nch w=1u l=180n
M1120 t421 nq1 0 0 nch w=1u l=180n
M1121 nw140 t420 vdd vdd pch w=2u l=180n
M1122 nw140 t420 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
CT422 t422 0 0.1f
M1123 t422 nw106 0 0 nch w=1u l=180n
M1124 t422 nq3 0 0 nch w=1u l=180n
CT423 t423 0 0.1f
M1125 t423 nw106 vdd vdd pch w=2u l=180n
M1126 t422 nq3 t423 vdd pch w=2u l=180n
M1127 nw141 t422 vdd vdd pch w=2u l=180n
M1128 nw141 t422 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
CT424 t424 0 0.1f
CT425 t425 0 0.1f
CT426 t426 0 0.1f
M1129 t424 nw108 vdd vdd pch w=2u l=180n
M1130 t424 nq5 vdd vdd pch w=2u l=180n
CT427 t427 0 0.1f
M1131 t424 nw108 t427 0 nch w=1u l=180n
M1132 t427 nq5 0 0 nch w=1u l=180n
M1133 t425 nw108 vdd vdd pch w=2u l=180n
M1134 t425 t424 vdd vdd pch w=2u l=180n
CT428 t428 0 0.1f
M1135 t425 nw108 t428 0 nch w=1u l=180n
M1136 t428 t424 0 0 nch w=1u l=180n
M1137 t426 nq5 vdd vdd pch w=2u l=180n
M1138 t426 t424 vdd vdd pch w=2u l=180n
CT429 t429 0 0.1f
M1139 t426 nq5 t429 0 nch w=1u l=180n
M1140 t429 t424 0 0 nch w=1u l=180n
M1141 nw142 t425 vdd vdd pch w=2u l=180n
M1142 nw142 t426 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1143 nw142 t425 t430 0 nch w=1u l=180n
M1144 t430 t426 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
M1145 nw143 nw110 vdd vdd pch w=2u l=180n
M1146 nw143 nq7 vdd vdd pch w=2u l=180n
CT431 t431 0 0.1f
M1147 nw143 nw110 t431 0 nch w=1u l=180n
M1148 t431 nq7 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
M1149 nw144 nw112 0 0 nch w=1u l=180n
M1150 nw144 nq9 0 0 nch w=1u l=180n
CT432 t432 0 0.1f
M1151 t432 nw112 vdd vdd pch w=2u l=180n
M1152 nw144 nq9 t432 vdd pch w=2u l=180n
Cnw144 nw144 0 2f
CT433 t433 0 0.1f
M1153 t433 nw114 vdd vdd pch w=2u l=180n
M1154 t433 nq11 vdd vdd pch w=2u l=180n
CT434 t434 0 0.1f
M1155 t433 nw114 t434 0 nch w=1u l=180n
M1156 t434 nq11 0 0 nch w=1u l=180n
M1157 nw145 t433 vdd vdd pch w=2u l=180n
M1158 nw145 t433 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
CT435 t435 0 0.1f
M1159 t435 nw116 0 0 nch w=1u l=180n
M1160 t435 nq13 0 0 nch w=1u l=180n
CT436 t436 0 0.1f
M1161 t436 nw116 vdd vdd pch w=2u l=180n
M1162 t435 nq13 t436 vdd pch w=2u l=180n
M1163 nw146 t435 vdd vdd pch w=2u l=180n
M1164 nw146 t435 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
CT437 t437 0 0.1f
CT438 t438 0 0.1f
CT439 t439 0 0.1f
M1165 t437 nw118 vdd vdd pch w=2u l=180n
M1166 t437 nq15 vdd vdd pch w=2u l=180n
CT440 t440 0 0.1f
M1167 t437 nw118 t440 0 nch w=1u l=180n
M1168 t440 nq15 0 0 nch w=1u l=180n
M1169 t438 nw118 vdd vdd pch w=2u l=180n
M1170 t438 t437 vdd vdd pch w=2u l=180n
CT441 t441 0 0.1f
M1171 t438 nw118 t441 0 nch w=1u l=180n
M1172 t441 t437 0 0 nch w=1u l=180n
M1173 t439 nq15 vdd vdd pch w=2u l=180n
M1174 t439 t437 vdd vdd pch w=2u l=180n
CT442 t442 0 0.1f
M1175 t439 nq15 t442 0 nch w=1u l=180n
M1176 t442 t437 0 0 nch w=1u l=180n
M1177 nw147 t438 vdd vdd pch w=2u l=180n
M1178 nw147 t439 vdd vdd pch w=2u l=180n
CT443 t443 0 0.1f
M1179 nw147 t438 t443 0 nch w=1u l=180n
M1180 t443 t439 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
M1181 nw148 nw120 vdd vdd pch w=2u l=180n
M1182 nw148 ni1 vdd vdd pch w=2u l=180n
CT444 t444 0 0.1f
M1183 nw148 nw120 t444 0 nch w=1u l=180n
M1184 t444 ni1 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
M1185 nw149 nw122 0 0 nch w=1u l=180n
M1186 nw149 ni3 0 0 nch w=1u l=180n
CT445 t445 0 0.1f
M1187 t445 nw122 vdd vdd pch w=2u l=180n
M1188 nw149 ni3 t445 vdd pch w=2u l=180n
Cnw149 nw149 0 2f
CT446 t446 0 0.1f
M1189 t446 nw124 vdd vdd pch w=2u l=180n
M1190 t446 ni5 vdd vdd pch w=2u l=180n
CT447 t447 0 0.1f
M1191 t446 nw124 t447 0 nch w=1u l=180n
M1192 t447 ni5 0 0 nch w=1u l=180n
M1193 nw150 t446 vdd vdd pch w=2u l=180n
M1194 nw150 t446 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
CT448 t448 0 0.1f
M1195 t448 nw126 0 0 nch w=1u l=180n
M1196 t448 ni7 0 0 nch w=1u l=180n
CT449 t449 0 0.1f
M1197 t449 nw126 vdd vdd pch w=2u l=180n
M1198 t448 ni7 t449 vdd pch w=2u l=180n
M1199 nw151 t448 vdd vdd pch w=2u l=180n
M1200 nw151 t448 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
CT450 t450 0 0.1f
CT451 t451 0 0.1f
CT452 t452 0 0.1f
M1201 t450 nw128 vdd vdd pch w=2u l=180n
M1202 t450 nw34 vdd vdd pch w=2u l=180n
CT453 t453 0 0.1f
M1203 t450 nw128 t453 0 nch w=1u l=180n
M1204 t453 nw34 0 0 nch w=1u l=180n
M1205 t451 nw128 vdd vdd pch w=2u l=180n
M1206 t451 t450 vdd vdd pch w=2u l=180n
CT454 t454 0 0.1f
M1207 t451 nw128 t454 0 nch w=1u l=180n
M1208 t454 t450 0 0 nch w=1u l=180n
M1209 t452 nw34 vdd vdd pch w=2u l=180n
M1210 t452 t450 vdd vdd pch w=2u l=180n
CT455 t455 0 0.1f
M1211 t452 nw34 t455 0 nch w=1u l=180n
M1212 t455 t450 0 0 nch w=1u l=180n
M1213 nw152 t451 vdd vdd pch w=2u l=180n
M1214 nw152 t452 vdd vdd pch w=2u l=180n
CT456 t456 0 0.1f
M1215 nw152 t451 t456 0 nch w=1u l=180n
M1216 t456 t452 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
M1217 nw153 nw130 vdd vdd pch w=2u l=180n
M1218 nw153 nw36 vdd vdd pch w=2u l=180n
CT457 t457 0 0.1f
M1219 nw153 nw130 t457 0 nch w=1u l=180n
M1220 t457 nw36 0 0 nch w=1u l=180n
Cnw153 nw153 0 2f
M1221 nw154 nw132 0 0 nch w=1u l=180n
M1222 nw154 nw38 0 0 nch w=1u l=180n
CT458 t458 0 0.1f
M1223 t458 nw132 vdd vdd pch w=2u l=180n
M1224 nw154 nw38 t458 vdd pch w=2u l=180n
Cnw154 nw154 0 2f
CT459 t459 0 0.1f
M1225 t459 nw134 vdd vdd pch w=2u l=180n
M1226 t459 nw40 vdd vdd pch w=2u l=180n
CT460 t460 0 0.1f
M1227 t459 nw134 t460 0 nch w=1u l=180n
M1228 t460 nw40 0 0 nch w=1u l=180n
M1229 nw155 t459 vdd vdd pch w=2u l=180n
M1230 nw155 t459 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
CT461 t461 0 0.1f
M1231 t461 nw136 0 0 nch w=1u l=180n
M1232 t461 nw42 0 0 nch w=1u l=180n
CT462 t462 0 0.1f
M1233 t462 nw136 vdd vdd pch w=2u l=180n
M1234 t461 nw42 t462 vdd pch w=2u l=180n
M1235 nw156 t461 vdd vdd pch w=2u l=180n
M1236 nw156 t461 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
CT463 t463 0 0.1f
CT464 t464 0 0.1f
CT465 t465 0 0.1f
M1237 t463 nw138 vdd vdd pch w=2u l=180n
M1238 t463 nw44 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1239 t463 nw138 t466 0 nch w=1u l=180n
M1240 t466 nw44 0 0 nch w=1u l=180n
M1241 t464 nw138 vdd vdd pch w=2u l=180n
M1242 t464 t463 vdd vdd pch w=2u l=180n
CT467 t467 0 0.1f
M1243 t464 nw138 t467 0 nch w=1u l=180n
M1244 t467 t463 0 0 nch w=1u l=180n
M1245 t465 nw44 vdd vdd pch w=2u l=180n
M1246 t465 t463 vdd vdd pch w=2u l=180n
CT468 t468 0 0.1f
M1247 t465 nw44 t468 0 nch w=1u l=180n
M1248 t468 t463 0 0 nch w=1u l=180n
M1249 nw157 t464 vdd vdd pch w=2u l=180n
M1250 nw157 t465 vdd vdd pch w=2u l=180n
CT469 t469 0 0.1f
M1251 nw157 t464 t469 0 nch w=1u l=180n
M1252 t469 t465 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
M1253 nw158 nw140 vdd vdd pch w=2u l=180n
M1254 nw158 nw46 vdd vdd pch w=2u l=180n
CT470 t470 0 0.1f
M1255 nw158 nw140 t470 0 nch w=1u l=180n
M1256 t470 nw46 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
M1257 nw159 nw142 0 0 nch w=1u l=180n
M1258 nw159 nw48 0 0 nch w=1u l=180n
CT471 t471 0 0.1f
M1259 t471 nw142 vdd vdd pch w=2u l=180n
M1260 nw159 nw48 t471 vdd pch w=2u l=180n
Cnw159 nw159 0 2f
CT472 t472 0 0.1f
M1261 t472 nw144 vdd vdd pch w=2u l=180n
M1262 t472 nw50 vdd vdd pch w=2u l=180n
CT473 t473 0 0.1f
M1263 t472 nw144 t473 0 nch w=1u l=180n
M1264 t473 nw50 0 0 nch w=1u l=180n
M1265 nw160 t472 vdd vdd pch w=2u l=180n
M1266 nw160 t472 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
CT474 t474 0 0.1f
M1267 t474 nw146 0 0 nch w=1u l=180n
M1268 t474 nw52 0 0 nch w=1u l=180n
CT475 t475 0 0.1f
M1269 t475 nw146 vdd vdd pch w=2u l=180n
M1270 t474 nw52 t475 vdd pch w=2u l=180n
M1271 nw161 t474 vdd vdd pch w=2u l=180n
M1272 nw161 t474 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
CT476 t476 0 0.1f
CT477 t477 0 0.1f
CT478 t478 0 0.1f
M1273 t476 nw148 vdd vdd pch w=2u l=180n
M1274 t476 nw54 vdd vdd pch w=2u l=180n
CT479 t479 0 0.1f
M1275 t476 nw148 t479 0 nch w=1u l=180n
M1276 t479 nw54 0 0 nch w=1u l=180n
M1277 t477 nw148 vdd vdd pch w=2u l=180n
M1278 t477 t476 vdd vdd pch w=2u l=180n
CT480 t480 0 0.1f
M1279 t477 nw148 t480 0 nch w=1u l=180n
M1280 t480 t476 0 0 nch w=1u l=180n
M1281 t478 nw54 vdd vdd pch w=2u l=180n
M1282 t478 t476 vdd vdd pch w=2u l=180n
CT481 t481 0 0.1f
M1283 t478 nw54 t481 0 nch w=1u l=180n
M1284 t481 t476 0 0 nch w=1u l=180n
M1285 nw162 t477 vdd vdd pch w=2u l=180n
M1286 nw162 t478 vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1287 nw162 t477 t482 0 nch w=1u l=180n
M1288 t482 t478 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
M1289 nw163 nw150 vdd vdd pch w=2u l=180n
M1290 nw163 nw56 vdd vdd pch w=2u l=180n
CT483 t483 0 0.1f
M1291 nw163 nw150 t483 0 nch w=1u l=180n
M1292 t483 nw56 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
M1293 nw164 nw152 0 0 nch w=1u l=180n
M1294 nw164 nw58 0 0 nch w=1u l=180n
CT484 t484 0 0.1f
M1295 t484 nw152 vdd vdd pch w=2u l=180n
M1296 nw164 nw58 t484 vdd pch w=2u l=180n
Cnw164 nw164 0 2f
CT485 t485 0 0.1f
M1297 t485 nw154 vdd vdd pch w=2u l=180n
M1298 t485 nw60 vdd vdd pch w=2u l=180n
CT486 t486 0 0.1f
M1299 t485 nw154 t486 0 nch w=1u l=180n
M1300 t486 nw60 0 0 nch w=1u l=180n
M1301 nw165 t485 vdd vdd pch w=2u l=180n
M1302 nw165 t485 0 0 nch w=1u l=180n
Cnw165 nw165 0 2f
CT487 t487 0 0.1f
M1303 t487 nw156 0 0 nch w=1u l=180n
M1304 t487 nw62 0 0 nch w=1u l=180n
CT488 t488 0 0.1f
M1305 t488 nw156 vdd vdd pch w=2u l=180n
M1306 t487 nw62 t488 vdd pch w=2u l=180n
M1307 nw166 t487 vdd vdd pch w=2u l=180n
M1308 nw166 t487 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
CT489 t489 0 0.1f
CT490 t490 0 0.1f
CT491 t491 0 0.1f
M1309 t489 nw158 vdd vdd pch w=2u l=180n
M1310 t489 nw64 vdd vdd pch w=2u l=180n
CT492 t492 0 0.1f
M1311 t489 nw158 t492 0 nch w=1u l=180n
M1312 t492 nw64 0 0 nch w=1u l=180n
M1313 t490 nw158 vdd vdd pch w=2u l=180n
M1314 t490 t489 vdd vdd pch w=2u l=180n
CT493 t493 0 0.1f
M1315 t490 nw158 t493 0 nch w=1u l=180n
M1316 t493 t489 0 0 nch w=1u l=180n
M1317 t491 nw64 vdd vdd pch w=2u l=180n
M1318 t491 t489 vdd vdd pch w=2u l=180n
CT494 t494 0 0.1f
M1319 t491 nw64 t494 0 nch w=1u l=180n
M1320 t494 t489 0 0 nch w=1u l=180n
M1321 nw167 t490 vdd vdd pch w=2u l=180n
M1322 nw167 t491 vdd vdd pch w=2u l=180n
CT495 t495 0 0.1f
M1323 nw167 t490 t495 0 nch w=1u l=180n
M1324 t495 t491 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
M1325 nw168 nw160 vdd vdd pch w=2u l=180n
M1326 nw168 nw66 vdd vdd pch w=2u l=180n
CT496 t496 0 0.1f
M1327 nw168 nw160 t496 0 nch w=1u l=180n
M1328 t496 nw66 0 0 nch w=1u l=180n
Cnw168 nw168 0 2f
M1329 nw169 nw162 0 0 nch w=1u l=180n
M1330 nw169 nw68 0 0 nch w=1u l=180n
CT497 t497 0 0.1f
M1331 t497 nw162 vdd vdd pch w=2u l=180n
M1332 nw169 nw68 t497 vdd pch w=2u l=180n
Cnw169 nw169 0 2f
CT498 t498 0 0.1f
M1333 t498 nw164 vdd vdd pch w=2u l=180n
M1334 t498 nw70 vdd vdd pch w=2u l=180n
CT499 t499 0 0.1f
M1335 t498 nw164 t499 0 nch w=1u l=180n
M1336 t499 nw70 0 0 nch w=1u l=180n
M1337 nw170 t498 vdd vdd pch w=2u l=180n
M1338 nw170 t498 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
CT500 t500 0 0.1f
M1339 t500 nw166 0 0 nch w=1u l=180n
M1340 t500 nw72 0 0 nch w=1u l=180n
CT501 t501 0 0.1f
M1341 t501 nw166 vdd vdd pch w=2u l=180n
M1342 t500 nw72 t501 vdd pch w=2u l=180n
M1343 nw171 t500 vdd vdd pch w=2u l=180n
M1344 nw171 t500 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
CT502 t502 0 0.1f
CT503 t503 0 0.1f
CT504 t504 0 0.1f
M1345 t502 nw168 vdd vdd pch w=2u l=180n
M1346 t502 nw74 vdd vdd pch w=2u l=180n
CT505 t505 0 0.1f
M1347 t502 nw168 t505 0 nch w=1u l=180n
M1348 t505 nw74 0 0 nch w=1u l=180n
M1349 t503 nw168 vdd vdd pch w=2u l=180n
M1350 t503 t502 vdd vdd pch w=2u l=180n
CT506 t506 0 0.1f
M1351 t503 nw168 t506 0 nch w=1u l=180n
M1352 t506 t502 0 0 nch w=1u l=180n
M1353 t504 nw74 vdd vdd pch w=2u l=180n
M1354 t504 t502 vdd vdd pch w=2u l=180n
CT507 t507 0 0.1f
M1355 t504 nw74 t507 0 nch w=1u l=180n
M1356 t507 t502 0 0 nch w=1u l=180n
M1357 nw172 t503 vdd vdd pch w=2u l=180n
M1358 nw172 t504 vdd vdd pch w=2u l=180n
CT508 t508 0 0.1f
M1359 nw172 t503 t508 0 nch w=1u l=180n
M1360 t508 t504 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
M1361 nw173 nw170 vdd vdd pch w=2u l=180n
M1362 nw173 nw76 vdd vdd pch w=2u l=180n
CT509 t509 0 0.1f
M1363 nw173 nw170 t509 0 nch w=1u l=180n
M1364 t509 nw76 0 0 nch w=1u l=180n
Cnw173 nw173 0 2f
M1365 nw174 nw172 0 0 nch w=1u l=180n
M1366 nw174 nw78 0 0 nch w=1u l=180n
CT510 t510 0 0.1f
M1367 t510 nw172 vdd vdd pch w=2u l=180n
M1368 nw174 nw78 t510 vdd pch w=2u l=180n
Cnw174 nw174 0 2f
CT511 t511 0 0.1f
M1369 t511 nw174 vdd vdd pch w=2u l=180n
M1370 t511 nw80 vdd vdd pch w=2u l=180n
CT512 t512 0 0.1f
M1371 t511 nw174 t512 0 nch w=1u l=180n
M1372 t512 nw80 0 0 nch w=1u l=180n
M1373 nw175 t511 vdd vdd pch w=2u l=180n
M1374 nw175 t511 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
CT513 t513 0 0.1f
M1375 t513 nq0 0 0 nch w=1u l=180n
M1376 t513 nw82 0 0 nch w=1u l=180n
CT514 t514 0 0.1f
M1377 t514 nq0 vdd vdd pch w=2u l=180n
M1378 t513 nw82 t514 vdd pch w=2u l=180n
M1379 nw176 t513 vdd vdd pch w=2u l=180n
M1380 nw176 t513 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
CT515 t515 0 0.1f
CT516 t516 0 0.1f
CT517 t517 0 0.1f
M1381 t515 nq1 vdd vdd pch w=2u l=180n
M1382 t515 nw84 vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1383 t515 nq1 t518 0 nch w=1u l=180n
M1384 t518 nw84 0 0 nch w=1u l=180n
M1385 t516 nq1 vdd vdd pch w=2u l=180n
M1386 t516 t515 vdd vdd pch w=2u l=180n
CT519 t519 0 0.1f
M1387 t516 nq1 t519 0 nch w=1u l=180n
M1388 t519 t515 0 0 nch w=1u l=180n
M1389 t517 nw84 vdd vdd pch w=2u l=180n
M1390 t517 t515 vdd vdd pch w=2u l=180n
CT520 t520 0 0.1f
M1391 t517 nw84 t520 0 nch w=1u l=180n
M1392 t520 t515 0 0 nch w=1u l=180n
M1393 nw177 t516 vdd vdd pch w=2u l=180n
M1394 nw177 t517 vdd vdd pch w=2u l=180n
CT521 t521 0 0.1f
M1395 nw177 t516 t521 0 nch w=1u l=180n
M1396 t521 t517 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
M1397 nw178 nq2 vdd vdd pch w=2u l=180n
M1398 nw178 nw86 vdd vdd pch w=2u l=180n
CT522 t522 0 0.1f
M1399 nw178 nq2 t522 0 nch w=1u l=180n
M1400 t522 nw86 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
M1401 nw179 nq3 0 0 nch w=1u l=180n
M1402 nw179 nw88 0 0 nch w=1u l=180n
CT523 t523 0 0.1f
M1403 t523 nq3 vdd vdd pch w=2u l=180n
M1404 nw179 nw88 t523 vdd pch w=2u l=180n
Cnw179 nw179 0 2f
CT524 t524 0 0.1f
M1405 t524 nq4 vdd vdd pch w=2u l=180n
M1406 t524 nw90 vdd vdd pch w=2u l=180n
CT525 t525 0 0.1f
M1407 t524 nq4 t525 0 nch w=1u l=180n
M1408 t525 nw90 0 0 nch w=1u l=180n
M1409 nw180 t524 vdd vdd pch w=2u l=180n
M1410 nw180 t524 0 0 nch w=1u l=180n
Cnw180 nw180 0 2f
CT526 t526 0 0.1f
M1411 t526 nq5 0 0 nch w=1u l=180n
M1412 t526 nw92 0 0 nch w=1u l=180n
CT527 t527 0 0.1f
M1413 t527 nq5 vdd vdd pch w=2u l=180n
M1414 t526 nw92 t527 vdd pch w=2u l=180n
M1415 nw181 t526 vdd vdd pch w=2u l=180n
M1416 nw181 t526 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
CT528 t528 0 0.1f
CT529 t529 0 0.1f
CT530 t530 0 0.1f
M1417 t528 nq6 vdd vdd pch w=2u l=180n
M1418 t528 nw94 vdd vdd pch w=2u l=180n
CT531 t531 0 0.1f
M1419 t528 nq6 t531 0 nch w=1u l=180n
M1420 t531 nw94 0 0 nch w=1u l=180n
M1421 t529 nq6 vdd vdd pch w=2u l=180n
M1422 t529 t528 vdd vdd pch w=2u l=180n
CT532 t532 0 0.1f
M1423 t529 nq6 t532 0 nch w=1u l=180n
M1424 t532 t528 0 0 nch w=1u l=180n
M1425 t530 nw94 vdd vdd pch w=2u l=180n
M1426 t530 t528 vdd vdd pch w=2u l=180n
CT533 t533 0 0.1f
M1427 t530 nw94 t533 0 nch w=1u l=180n
M1428 t533 t528 0 0 nch w=1u l=180n
M1429 nw182 t529 vdd vdd pch w=2u l=180n
M1430 nw182 t530 vdd vdd pch w=2u l=180n
CT534 t534 0 0.1f
M1431 nw182 t529 t534 0 nch w=1u l=180n
M1432 t534 t530 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
M1433 nw183 nq7 vdd vdd pch w=2u l=180n
M1434 nw183 nw96 vdd vdd pch w=2u l=180n
CT535 t535 0 0.1f
M1435 nw183 nq7 t535 0 nch w=1u l=180n
M1436 t535 nw96 0 0 nch w=1u l=180n
Cnw183 nw183 0 2f
M1437 nw184 nq8 0 0 nch w=1u l=180n
M1438 nw184 nw98 0 0 nch w=1u l=180n
CT536 t536 0 0.1f
M1439 t536 nq8 vdd vdd pch w=2u l=180n
M1440 nw184 nw98 t536 vdd pch w=2u l=180n
Cnw184 nw184 0 2f
CT537 t537 0 0.1f
M1441 t537 nq9 vdd vdd pch w=2u l=180n
M1442 t537 nw100 vdd vdd pch w=2u l=180n
CT538 t538 0 0.1f
M1443 t537 nq9 t538 0 nch w=1u l=180n
M1444 t538 nw100 0 0 nch w=1u l=180n
M1445 nw185 t537 vdd vdd pch w=2u l=180n
M1446 nw185 t537 0 0 nch w=1u l=180n
Cnw185 nw185 0 2f
CT539 t539 0 0.1f
M1447 t539 nq10 0 0 nch w=1u l=180n
M1448 t539 nw102 0 0 nch w=1u l=180n
CT540 t540 0 0.1f
M1449 t540 nq10 vdd vdd pch w=2u l=180n
M1450 t539 nw102 t540 vdd pch w=2u l=180n
M1451 nw186 t539 vdd vdd pch w=2u l=180n
M1452 nw186 t539 0 0 nch w=1u l=180n
Cnw186 nw186 0 2f
CT541 t541 0 0.1f
CT542 t542 0 0.1f
CT543 t543 0 0.1f
M1453 t541 nq11 vdd vdd pch w=2u l=180n
M1454 t541 nw104 vdd vdd pch w=2u l=180n
CT544 t544 0 0.1f
M1455 t541 nq11 t544 0 nch w=1u l=180n
M1456 t544 nw104 0 0 nch w=1u l=180n
M1457 t542 nq11 vdd vdd pch w=2u l=180n
M1458 t542 t541 vdd vdd pch w=2u l=180n
CT545 t545 0 0.1f
M1459 t542 nq11 t545 0 nch w=1u l=180n
M1460 t545 t541 0 0 nch w=1u l=180n
M1461 t543 nw104 vdd vdd pch w=2u l=180n
M1462 t543 t541 vdd vdd pch w=2u l=180n
CT546 t546 0 0.1f
M1463 t543 nw104 t546 0 nch w=1u l=180n
M1464 t546 t541 0 0 nch w=1u l=180n
M1465 nw187 t542 vdd vdd pch w=2u l=180n
M1466 nw187 t543 vdd vdd pch w=2u l=180n
CT547 t547 0 0.1f
M1467 nw187 t542 t547 0 nch w=1u l=180n
M1468 t547 t543 0 0 nch w=1u l=180n
Cnw187 nw187 0 2f
M1469 nw188 nq12 vdd vdd pch w=2u l=180n
M1470 nw188 nw106 vdd vdd pch w=2u l=180n
CT548 t548 0 0.1f
M1471 nw188 nq12 t548 0 nch w=1u l=180n
M1472 t548 nw106 0 0 nch w=1u l=180n
Cnw188 nw188 0 2f
M1473 nw189 nq13 0 0 nch w=1u l=180n
M1474 nw189 nw108 0 0 nch w=1u l=180n
CT549 t549 0 0.1f
M1475 t549 nq13 vdd vdd pch w=2u l=180n
M1476 nw189 nw108 t549 vdd pch w=2u l=180n
Cnw189 nw189 0 2f
CT550 t550 0 0.1f
M1477 t550 nq14 vdd vdd pch w=2u l=180n
M1478 t550 nw110 vdd vdd pch w=2u l=180n
CT551 t551 0 0.1f
M1479 t550 nq14 t551 0 nch w=1u l=180n
M1480 t551 nw110 0 0 nch w=1u l=180n
M1481 nw190 t550 vdd vdd pch w=2u l=180n
M1482 nw190 t550 0 0 nch w=1u l=180n
Cnw190 nw190 0 2f
CT552 t552 0 0.1f
M1483 t552 nq15 0 0 nch w=1u l=180n
M1484 t552 nw112 0 0 nch w=1u l=180n
CT553 t553 0 0.1f
M1485 t553 nq15 vdd vdd pch w=2u l=180n
M1486 t552 nw112 t553 vdd pch w=2u l=180n
M1487 nw191 t552 vdd vdd pch w=2u l=180n
M1488 nw191 t552 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
CT554 t554 0 0.1f
CT555 t555 0 0.1f
CT556 t556 0 0.1f
M1489 t554 ni0 vdd vdd pch w=2u l=180n
M1490 t554 nw114 vdd vdd pch w=2u l=180n
CT557 t557 0 0.1f
M1491 t554 ni0 t557 0 nch w=1u l=180n
M1492 t557 nw114 0 0 nch w=1u l=180n
M1493 t555 ni0 vdd vdd pch w=2u l=180n
M1494 t555 t554 vdd vdd pch w=2u l=180n
CT558 t558 0 0.1f
M1495 t555 ni0 t558 0 nch w=1u l=180n
M1496 t558 t554 0 0 nch w=1u l=180n
M1497 t556 nw114 vdd vdd pch w=2u l=180n
M1498 t556 t554 vdd vdd pch w=2u l=180n
CT559 t559 0 0.1f
M1499 t556 nw114 t559 0 nch w=1u l=180n
M1500 t559 t554 0 0 nch w=1u l=180n
M1501 nw192 t555 vdd vdd pch w=2u l=180n
M1502 nw192 t556 vdd vdd pch w=2u l=180n
CT560 t560 0 0.1f
M1503 nw192 t555 t560 0 nch w=1u l=180n
M1504 t560 t556 0 0 nch w=1u l=180n
Cnw192 nw192 0 2f
M1505 nw193 ni1 vdd vdd pch w=2u l=180n
M1506 nw193 nw116 vdd vdd pch w=2u l=180n
CT561 t561 0 0.1f
M1507 nw193 ni1 t561 0 nch w=1u l=180n
M1508 t561 nw116 0 0 nch w=1u l=180n
Cnw193 nw193 0 2f
M1509 nw194 ni2 0 0 nch w=1u l=180n
M1510 nw194 nw118 0 0 nch w=1u l=180n
CT562 t562 0 0.1f
M1511 t562 ni2 vdd vdd pch w=2u l=180n
M1512 nw194 nw118 t562 vdd pch w=2u l=180n
Cnw194 nw194 0 2f
CT563 t563 0 0.1f
M1513 t563 ni3 vdd vdd pch w=2u l=180n
M1514 t563 nw120 vdd vdd pch w=2u l=180n
CT564 t564 0 0.1f
M1515 t563 ni3 t564 0 nch w=1u l=180n
M1516 t564 nw120 0 0 nch w=1u l=180n
M1517 nw195 t563 vdd vdd pch w=2u l=180n
M1518 nw195 t563 0 0 nch w=1u l=180n
Cnw195 nw195 0 2f
CT565 t565 0 0.1f
M1519 t565 ni4 0 0 nch w=1u l=180n
M1520 t565 nw122 0 0 nch w=1u l=180n
CT566 t566 0 0.1f
M1521 t566 ni4 vdd vdd pch w=2u l=180n
M1522 t565 nw122 t566 vdd pch w=2u l=180n
M1523 nw196 t565 vdd vdd pch w=2u l=180n
M1524 nw196 t565 0 0 nch w=1u l=180n
Cnw196 nw196 0 2f
CT567 t567 0 0.1f
CT568 t568 0 0.1f
CT569 t569 0 0.1f
M1525 t567 ni5 vdd vdd pch w=2u l=180n
M1526 t567 nw124 vdd vdd pch w=2u l=180n
CT570 t570 0 0.1f
M1527 t567 ni5 t570 0 nch w=1u l=180n
M1528 t570 nw124 0 0 nch w=1u l=180n
M1529 t568 ni5 vdd vdd pch w=2u l=180n
M1530 t568 t567 vdd vdd pch w=2u l=180n
CT571 t571 0 0.1f
M1531 t568 ni5 t571 0 nch w=1u l=180n
M1532 t571 t567 0 0 nch w=1u l=180n
M1533 t569 nw124 vdd vdd pch w=2u l=180n
M1534 t569 t567 vdd vdd pch w=2u l=180n
CT572 t572 0 0.1f
M1535 t569 nw124 t572 0 nch w=1u l=180n
M1536 t572 t567 0 0 nch w=1u l=180n
M1537 nw197 t568 vdd vdd pch w=2u l=180n
M1538 nw197 t569 vdd vdd pch w=2u l=180n
CT573 t573 0 0.1f
M1539 nw197 t568 t573 0 nch w=1u l=180n
M1540 t573 t569 0 0 nch w=1u l=180n
Cnw197 nw197 0 2f
M1541 nw198 ni6 vdd vdd pch w=2u l=180n
M1542 nw198 nw126 vdd vdd pch w=2u l=180n
CT574 t574 0 0.1f
M1543 nw198 ni6 t574 0 nch w=1u l=180n
M1544 t574 nw126 0 0 nch w=1u l=180n
Cnw198 nw198 0 2f
M1545 nw199 ni7 0 0 nch w=1u l=180n
M1546 nw199 nw128 0 0 nch w=1u l=180n
CT575 t575 0 0.1f
M1547 t575 ni7 vdd vdd pch w=2u l=180n
M1548 nw199 nw128 t575 vdd pch w=2u l=180n
Cnw199 nw199 0 2f
CT576 t576 0 0.1f
M1549 t576 nw33 vdd vdd pch w=2u l=180n
M1550 t576 nw130 vdd vdd pch w=2u l=180n
CT577 t577 0 0.1f
M1551 t576 nw33 t577 0 nch w=1u l=180n
M1552 t577 nw130 0 0 nch w=1u l=180n
M1553 nw200 t576 vdd vdd pch w=2u l=180n
M1554 nw200 t576 0 0 nch w=1u l=180n
Cnw200 nw200 0 2f
CT578 t578 0 0.1f
M1555 t578 nw34 0 0 nch w=1u l=180n
M1556 t578 nw132 0 0 nch w=1u l=180n
CT579 t579 0 0.1f
M1557 t579 nw34 vdd vdd pch w=2u l=180n
M1558 t578 nw132 t579 vdd pch w=2u l=180n
M1559 nw201 t578 vdd vdd pch w=2u l=180n
M1560 nw201 t578 0 0 nch w=1u l=180n
Cnw201 nw201 0 2f
CT580 t580 0 0.1f
CT581 t581 0 0.1f
CT582 t582 0 0.1f
M1561 t580 nw35 vdd vdd pch w=2u l=180n
M1562 t580 nw134 vdd vdd pch w=2u l=180n
CT583 t583 0 0.1f
M1563 t580 nw35 t583 0 nch w=1u l=180n
M1564 t583 nw134 0 0 nch w=1u l=180n
M1565 t581 nw35 vdd vdd pch w=2u l=180n
M1566 t581 t580 vdd vdd pch w=2u l=180n
CT584 t584 0 0.1f
M1567 t581 nw35 t584 0 nch w=1u l=180n
M1568 t584 t580 0 0 nch w=1u l=180n
M1569 t582 nw134 vdd vdd pch w=2u l=180n
M1570 t582 t580 vdd vdd pch w=2u l=180n
CT585 t585 0 0.1f
M1571 t582 nw134 t585 0 nch w=1u l=180n
M1572 t585 t580 0 0 nch w=1u l=180n
M1573 nw202 t581 vdd vdd pch w=2u l=180n
M1574 nw202 t582 vdd vdd pch w=2u l=180n
CT586 t586 0 0.1f
M1575 nw202 t581 t586 0 nch w=1u l=180n
M1576 t586 t582 0 0 nch w=1u l=180n
Cnw202 nw202 0 2f
M1577 nw203 nw36 vdd vdd pch w=2u l=180n
M1578 nw203 nw136 vdd vdd pch w=2u l=180n
CT587 t587 0 0.1f
M1579 nw203 nw36 t587 0 nch w=1u l=180n
M1580 t587 nw136 0 0 nch w=1u l=180n
Cnw203 nw203 0 2f
M1581 nw204 nw37 0 0 nch w=1u l=180n
M1582 nw204 nw138 0 0 nch w=1u l=180n
CT588 t588 0 0.1f
M1583 t588 nw37 vdd vdd pch w=2u l=180n
M1584 nw204 nw138 t588 vdd pch w=2u l=180n
Cnw204 nw204 0 2f
CT589 t589 0 0.1f
M1585 t589 nw38 vdd vdd pch w=2u l=180n
M1586 t589 nw140 vdd vdd pch w=2u l=180n
CT590 t590 0 0.1f
M1587 t589 nw38 t590 0 nch w=1u l=180n
M1588 t590 nw140 0 0 nch w=1u l=180n
M1589 nw205 t589 vdd vdd pch w=2u l=180n
M1590 nw205 t589 0 0 nch w=1u l=180n
Cnw205 nw205 0 2f
CT591 t591 0 0.1f
M1591 t591 nw39 0 0 nch w=1u l=180n
M1592 t591 nw142 0 0 nch w=1u l=180n
CT592 t592 0 0.1f
M1593 t592 nw39 vdd vdd pch w=2u l=180n
M1594 t591 nw142 t592 vdd pch w=2u l=180n
M1595 nw206 t591 vdd vdd pch w=2u l=180n
M1596 nw206 t591 0 0 nch w=1u l=180n
Cnw206 nw206 0 2f
CT593 t593 0 0.1f
CT594 t594 0 0.1f
CT595 t595 0 0.1f
M1597 t593 nw40 vdd vdd pch w=2u l=180n
M1598 t593 nw144 vdd vdd pch w=2u l=180n
CT596 t596 0 0.1f
M1599 t593 nw40 t596 0 nch w=1u l=180n
M1600 t596 nw144 0 0 nch w=1u l=180n
M1601 t594 nw40 vdd vdd pch w=2u l=180n
M1602 t594 t593 vdd vdd pch w=2u l=180n
CT597 t597 0 0.1f
M1603 t594 nw40 t597 0 nch w=1u l=180n
M1604 t597 t593 0 0 nch w=1u l=180n
M1605 t595 nw144 vdd vdd pch w=2u l=180n
M1606 t595 t593 vdd vdd pch w=2u l=180n
CT598 t598 0 0.1f
M1607 t595 nw144 t598 0 nch w=1u l=180n
M1608 t598 t593 0 0 nch w=1u l=180n
M1609 nw207 t594 vdd vdd pch w=2u l=180n
M1610 nw207 t595 vdd vdd pch w=2u l=180n
CT599 t599 0 0.1f
M1611 nw207 t594 t599 0 nch w=1u l=180n
M1612 t599 t595 0 0 nch w=1u l=180n
Cnw207 nw207 0 2f
M1613 nw208 nw41 vdd vdd pch w=2u l=180n
M1614 nw208 nw146 vdd vdd pch w=2u l=180n
CT600 t600 0 0.1f
M1615 nw208 nw41 t600 0 nch w=1u l=180n
M1616 t600 nw146 0 0 nch w=1u l=180n
Cnw208 nw208 0 2f
M1617 nw209 nw42 0 0 nch w=1u l=180n
M1618 nw209 nw148 0 0 nch w=1u l=180n
CT601 t601 0 0.1f
M1619 t601 nw42 vdd vdd pch w=2u l=180n
M1620 nw209 nw148 t601 vdd pch w=2u l=180n
Cnw209 nw209 0 2f
CT602 t602 0 0.1f
M1621 t602 nw43 vdd vdd pch w=2u l=180n
M1622 t602 nw150 vdd vdd pch w=2u l=180n
CT603 t603 0 0.1f
M1623 t602 nw43 t603 0 nch w=1u l=180n
M1624 t603 nw150 0 0 nch w=1u l=180n
M1625 nw210 t602 vdd vdd pch w=2u l=180n
M1626 nw210 t602 0 0 nch w=1u l=180n
Cnw210 nw210 0 2f
CT604 t604 0 0.1f
M1627 t604 nw44 0 0 nch w=1u l=180n
M1628 t604 nw152 0 0 nch w=1u l=180n
CT605 t605 0 0.1f
M1629 t605 nw44 vdd vdd pch w=2u l=180n
M1630 t604 nw152 t605 vdd pch w=2u l=180n
M1631 nw211 t604 vdd vdd pch w=2u l=180n
M1632 nw211 t604 0 0 nch w=1u l=180n
Cnw211 nw211 0 2f
CT606 t606 0 0.1f
CT607 t607 0 0.1f
CT608 t608 0 0.1f
M1633 t606 nw45 vdd vdd pch w=2u l=180n
M1634 t606 nw154 vdd vdd pch w=2u l=180n
CT609 t609 0 0.1f
M1635 t606 nw45 t609 0 nch w=1u l=180n
M1636 t609 nw154 0 0 nch w=1u l=180n
M1637 t607 nw45 vdd vdd pch w=2u l=180n
M1638 t607 t606 vdd vdd pch w=2u l=180n
CT610 t610 0 0.1f
M1639 t607 nw45 t610 0 nch w=1u l=180n
M1640 t610 t606 0 0 nch w=1u l=180n
M1641 t608 nw154 vdd vdd pch w=2u l=180n
M1642 t608 t606 vdd vdd pch w=2u l=180n
CT611 t611 0 0.1f
M1643 t608 nw154 t611 0 nch w=1u l=180n
M1644 t611 t606 0 0 nch w=1u l=180n
M1645 nw212 t607 vdd vdd pch w=2u l=180n
M1646 nw212 t608 vdd vdd pch w=2u l=180n
CT612 t612 0 0.1f
M1647 nw212 t607 t612 0 nch w=1u l=180n
M1648 t612 t608 0 0 nch w=1u l=180n
Cnw212 nw212 0 2f
M1649 nw213 nw46 vdd vdd pch w=2u l=180n
M1650 nw213 nw156 vdd vdd pch w=2u l=180n
CT613 t613 0 0.1f
M1651 nw213 nw46 t613 0 nch w=1u l=180n
M1652 t613 nw156 0 0 nch w=1u l=180n
Cnw213 nw213 0 2f
M1653 nw214 nw47 0 0 nch w=1u l=180n
M1654 nw214 nw158 0 0 nch w=1u l=180n
CT614 t614 0 0.1f
M1655 t614 nw47 vdd vdd pch w=2u l=180n
M1656 nw214 nw158 t614 vdd pch w=2u l=180n
Cnw214 nw214 0 2f
CT615 t615 0 0.1f
M1657 t615 nw48 vdd vdd pch w=2u l=180n
M1658 t615 nw160 vdd vdd pch w=2u l=180n
CT616 t616 0 0.1f
M1659 t615 nw48 t616 0 nch w=1u l=180n
M1660 t616 nw160 0 0 nch w=1u l=180n
M1661 nw215 t615 vdd vdd pch w=2u l=180n
M1662 nw215 t615 0 0 nch w=1u l=180n
Cnw215 nw215 0 2f
CT617 t617 0 0.1f
M1663 t617 nw49 0 0 nch w=1u l=180n
M1664 t617 nw162 0 0 nch w=1u l=180n
CT618 t618 0 0.1f
M1665 t618 nw49 vdd vdd pch w=2u l=180n
M1666 t617 nw162 t618 vdd pch w=2u l=180n
M1667 nw216 t617 vdd vdd pch w=2u l=180n
M1668 nw216 t617 0 0 nch w=1u l=180n
Cnw216 nw216 0 2f
CT619 t619 0 0.1f
CT620 t620 0 0.1f
CT621 t621 0 0.1f
M1669 t619 nw50 vdd vdd pch w=2u l=180n
M1670 t619 nw164 vdd vdd pch w=2u l=180n
CT622 t622 0 0.1f
M1671 t619 nw50 t622 0 nch w=1u l=180n
M1672 t622 nw164 0 0 nch w=1u l=180n
M1673 t620 nw50 vdd vdd pch w=2u l=180n
M1674 t620 t619 vdd vdd pch w=2u l=180n
CT623 t623 0 0.1f
M1675 t620 nw50 t623 0 nch w=1u l=180n
M1676 t623 t619 0 0 nch w=1u l=180n
M1677 t621 nw164 vdd vdd pch w=2u l=180n
M1678 t621 t619 vdd vdd pch w=2u l=180n
CT624 t624 0 0.1f
M1679 t621 nw164 t624 0 nch w=1u l=180n
M1680 t624 t619 0 0 nch w=1u l=180n
M1681 nw217 t620 vdd vdd pch w=2u l=180n
M1682 nw217 t621 vdd vdd pch w=2u l=180n
CT625 t625 0 0.1f
M1683 nw217 t620 t625 0 nch w=1u l=180n
M1684 t625 t621 0 0 nch w=1u l=180n
Cnw217 nw217 0 2f
M1685 nw218 nw51 vdd vdd pch w=2u l=180n
M1686 nw218 nw166 vdd vdd pch w=2u l=180n
CT626 t626 0 0.1f
M1687 nw218 nw51 t626 0 nch w=1u l=180n
M1688 t626 nw166 0 0 nch w=1u l=180n
Cnw218 nw218 0 2f
M1689 nw219 nw52 0 0 nch w=1u l=180n
M1690 nw219 nw168 0 0 nch w=1u l=180n
CT627 t627 0 0.1f
M1691 t627 nw52 vdd vdd pch w=2u l=180n
M1692 nw219 nw168 t627 vdd pch w=2u l=180n
Cnw219 nw219 0 2f
CT628 t628 0 0.1f
M1693 t628 nw53 vdd vdd pch w=2u l=180n
M1694 t628 nw170 vdd vdd pch w=2u l=180n
CT629 t629 0 0.1f
M1695 t628 nw53 t629 0 nch w=1u l=180n
M1696 t629 nw170 0 0 nch w=1u l=180n
M1697 nw220 t628 vdd vdd pch w=2u l=180n
M1698 nw220 t628 0 0 nch w=1u l=180n
Cnw220 nw220 0 2f
CT630 t630 0 0.1f
M1699 t630 nw54 0 0 nch w=1u l=180n
M1700 t630 nw172 0 0 nch w=1u l=180n
CT631 t631 0 0.1f
M1701 t631 nw54 vdd vdd pch w=2u l=180n
M1702 t630 nw172 t631 vdd pch w=2u l=180n
M1703 nw221 t630 vdd vdd pch w=2u l=180n
M1704 nw221 t630 0 0 nch w=1u l=180n
Cnw221 nw221 0 2f
CT632 t632 0 0.1f
CT633 t633 0 0.1f
CT634 t634 0 0.1f
M1705 t632 nw55 vdd vdd pch w=2u l=180n
M1706 t632 nw174 vdd vdd pch w=2u l=180n
CT635 t635 0 0.1f
M1707 t632 nw55 t635 0 nch w=1u l=180n
M1708 t635 nw174 0 0 nch w=1u l=180n
M1709 t633 nw55 vdd vdd pch w=2u l=180n
M1710 t633 t632 vdd vdd pch w=2u l=180n
CT636 t636 0 0.1f
M1711 t633 nw55 t636 0 nch w=1u l=180n
M1712 t636 t632 0 0 nch w=1u l=180n
M1713 t634 nw174 vdd vdd pch w=2u l=180n
M1714 t634 t632 vdd vdd pch w=2u l=180n
CT637 t637 0 0.1f
M1715 t634 nw174 t637 0 nch w=1u l=180n
M1716 t637 t632 0 0 nch w=1u l=180n
M1717 nw222 t633 vdd vdd pch w=2u l=180n
M1718 nw222 t634 vdd vdd pch w=2u l=180n
CT638 t638 0 0.1f
M1719 nw222 t633 t638 0 nch w=1u l=180n
M1720 t638 t634 0 0 nch w=1u l=180n
Cnw222 nw222 0 2f
M1721 nw223 nw56 vdd vdd pch w=2u l=180n
M1722 nw223 nw176 vdd vdd pch w=2u l=180n
CT639 t639 0 0.1f
M1723 nw223 nw56 t639 0 nch w=1u l=180n
M1724 t639 nw176 0 0 nch w=1u l=180n
Cnw223 nw223 0 2f
M1725 nw224 nw57 0 0 nch w=1u l=180n
M1726 nw224 nw178 0 0 nch w=1u l=180n
CT640 t640 0 0.1f
M1727 t640 nw57 vdd vdd pch w=2u l=180n
M1728 nw224 nw178 t640 vdd pch w=2u l=180n
Cnw224 nw224 0 2f
CT641 t641 0 0.1f
M1729 t641 nw58 vdd vdd pch w=2u l=180n
M1730 t641 nw180 vdd vdd pch w=2u l=180n
CT642 t642 0 0.1f
M1731 t641 nw58 t642 0 nch w=1u l=180n
M1732 t642 nw180 0 0 nch w=1u l=180n
M1733 nw225 t641 vdd vdd pch w=2u l=180n
M1734 nw225 t641 0 0 nch w=1u l=180n
Cnw225 nw225 0 2f
CT643 t643 0 0.1f
M1735 t643 nw59 0 0 nch w=1u l=180n
M1736 t643 nw182 0 0 nch w=1u l=180n
CT644 t644 0 0.1f
M1737 t644 nw59 vdd vdd pch w=2u l=180n
M1738 t643 nw182 t644 vdd pch w=2u l=180n
M1739 nw226 t643 vdd vdd pch w=2u l=180n
M1740 nw226 t643 0 0 nch w=1u l=180n
Cnw226 nw226 0 2f
CT645 t645 0 0.1f
CT646 t646 0 0.1f
CT647 t647 0 0.1f
M1741 t645 nw60 vdd vdd pch w=2u l=180n
M1742 t645 nw184 vdd vdd pch w=2u l=180n
CT648 t648 0 0.1f
M1743 t645 nw60 t648 0 nch w=1u l=180n
M1744 t648 nw184 0 0 nch w=1u l=180n
M1745 t646 nw60 vdd vdd pch w=2u l=180n
M1746 t646 t645 vdd vdd pch w=2u l=180n
CT649 t649 0 0.1f
M1747 t646 nw60 t649 0 nch w=1u l=180n
M1748 t649 t645 0 0 nch w=1u l=180n
M1749 t647 nw184 vdd vdd pch w=2u l=180n
M1750 t647 t645 vdd vdd pch w=2u l=180n
CT650 t650 0 0.1f
M1751 t647 nw184 t650 0 nch w=1u l=180n
M1752 t650 t645 0 0 nch w=1u l=180n
M1753 nw227 t646 vdd vdd pch w=2u l=180n
M1754 nw227 t647 vdd vdd pch w=2u l=180n
CT651 t651 0 0.1f
M1755 nw227 t646 t651 0 nch w=1u l=180n
M1756 t651 t647 0 0 nch w=1u l=180n
Cnw227 nw227 0 2f
M1757 nw228 nw61 vdd vdd pch w=2u l=180n
M1758 nw228 nw186 vdd vdd pch w=2u l=180n
CT652 t652 0 0.1f
M1759 nw228 nw61 t652 0 nch w=1u l=180n
M1760 t652 nw186 0 0 nch w=1u l=180n
Cnw228 nw228 0 2f
M1761 nw229 nw62 0 0 nch w=1u l=180n
M1762 nw229 nw188 0 0 nch w=1u l=180n
CT653 t653 0 0.1f
M1763 t653 nw62 vdd vdd pch w=2u l=180n
M1764 nw229 nw188 t653 vdd pch w=2u l=180n
Cnw229 nw229 0 2f
CT654 t654 0 0.1f
M1765 t654 nw63 vdd vdd pch w=2u l=180n
M1766 t654 nw190 vdd vdd pch w=2u l=180n
CT655 t655 0 0.1f
M1767 t654 nw63 t655 0 nch w=1u l=180n
M1768 t655 nw190 0 0 nch w=1u l=180n
M1769 nw230 t654 vdd vdd pch w=2u l=180n
M1770 nw230 t654 0 0 nch w=1u l=180n
Cnw230 nw230 0 2f
CT656 t656 0 0.1f
M1771 t656 nw64 0 0 nch w=1u l=180n
M1772 t656 nw192 0 0 nch w=1u l=180n
CT657 t657 0 0.1f
M1773 t657 nw64 vdd vdd pch w=2u l=180n
M1774 t656 nw192 t657 vdd pch w=2u l=180n
M1775 nw231 t656 vdd vdd pch w=2u l=180n
M1776 nw231 t656 0 0 nch w=1u l=180n
Cnw231 nw231 0 2f
CT658 t658 0 0.1f
CT659 t659 0 0.1f
CT660 t660 0 0.1f
M1777 t658 nw65 vdd vdd pch w=2u l=180n
M1778 t658 nw194 vdd vdd pch w=2u l=180n
CT661 t661 0 0.1f
M1779 t658 nw65 t661 0 nch w=1u l=180n
M1780 t661 nw194 0 0 nch w=1u l=180n
M1781 t659 nw65 vdd vdd pch w=2u l=180n
M1782 t659 t658 vdd vdd pch w=2u l=180n
CT662 t662 0 0.1f
M1783 t659 nw65 t662 0 nch w=1u l=180n
M1784 t662 t658 0 0 nch w=1u l=180n
M1785 t660 nw194 vdd vdd pch w=2u l=180n
M1786 t660 t658 vdd vdd pch w=2u l=180n
CT663 t663 0 0.1f
M1787 t660 nw194 t663 0 nch w=1u l=180n
M1788 t663 t658 0 0 nch w=1u l=180n
M1789 nw232 t659 vdd vdd pch w=2u l=180n
M1790 nw232 t660 vdd vdd pch w=2u l=180n
CT664 t664 0 0.1f
M1791 nw232 t659 t664 0 nch w=1u l=180n
M1792 t664 t660 0 0 nch w=1u l=180n
Cnw232 nw232 0 2f
CT665 t665 0 0.1f
M1793 t665 nw232 vdd vdd pch w=2u l=180n
M1794 t665 nw232 0 0 nch w=1u l=180n
M1795 no0 t665 vdd vdd pch w=2u l=180n
M1796 no0 t665 0 0 nch w=1u l=180n
Cno0 no0 0 2f
CT666 t666 0 0.1f
M1797 t666 nw231 vdd vdd pch w=2u l=180n
M1798 t666 nw231 0 0 nch w=1u l=180n
M1799 no1 t666 vdd vdd pch w=2u l=180n
M1800 no1 t666 0 0 nch w=1u l=180n
Cno1 no1 0 2f
CT667 t667 0 0.1f
M1801 t667 nw230 vdd vdd pch w=2u l=180n
M1802 t667 nw230 0 0 nch w=1u l=180n
M1803 no2 t667 vdd vdd pch w=2u l=180n
M1804 no2 t667 0 0 nch w=1u l=180n
Cno2 no2 0 2f
CT668 t668 0 0.1f
M1805 t668 nw229 vdd vdd pch w=2u l=180n
M1806 t668 nw229 0 0 nch w=1u l=180n
M1807 no3 t668 vdd vdd pch w=2u l=180n
M1808 no3 t668 0 0 nch w=1u l=180n
Cno3 no3 0 2f
CT669 t669 0 0.1f
M1809 t669 nw228 vdd vdd pch w=2u l=180n
M1810 t669 nw228 0 0 nch w=1u l=180n
M1811 no4 t669 vdd vdd pch w=2u l=180n
M1812 no4 t669 0 0 nch w=1u l=180n
Cno4 no4 0 2f
CT670 t670 0 0.1f
M1813 t670 nw227 vdd vdd pch w=2u l=180n
M1814 t670 nw227 0 0 nch w=1u l=180n
M1815 no5 t670 vdd vdd pch w=2u l=180n
M1816 no5 t670 0 0 nch w=1u l=180n
Cno5 no5 0 2f
CT671 t671 0 0.1f
M1817 t671 nw226 vdd vdd pch w=2u l=180n
M1818 t671 nw226 0 0 nch w=1u l=180n
M1819 no6 t671 vdd vdd pch w=2u l=180n
M1820 no6 t671 0 0 nch w=1u l=180n
Cno6 no6 0 2f
CT672 t672 0 0.1f
M1821 t672 nw225 vdd vdd pch w=2u l=180n
M1822 t672 nw225 0 0 nch w=1u l=180n
M1823 no7 t672 vdd vdd pch w=2u l=180n
M1824 no7 t672 0 0 nch w=1u l=180n
Cno7 no7 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nw1 nw3 nw5 nw7 nw9 nw11 nw13 nw15 nw17 nw19 nw21 nw23 nw25 nw27 nw29 nw31 no0 no1 no2 no3 no4 no5 no6 no7
.end
